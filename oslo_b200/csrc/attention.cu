// Flash-style attention (forward, backward) and single-query decode attention.
//
// Scores never touch global memory: each CTA streams 64-wide blocks of the other operand through
// shared memory (cp.async, padded rows so ldmatrix is bank-conflict free) and keeps its output
// accumulators in registers. Masks are computed from indices: causal with a query offset
// (Sk - Sq, so the same kernel serves prefill with a prefix cache), GPT-Neo's sliding window
// (q_pos - window < k_pos <= q_pos; blocks wholly outside the window are skipped), and an optional
// key-padding byte mask. The backward is split in two passes that both recompute the probabilities from the
// saved log-sum-exp: a dQ pass (one CTA per query block, same shape as the forward) and a dK/dV pass
// (one CTA per key block, transposed orientation), so no atomics and no shared-memory transposes
// are needed and results are bitwise repeatable.
//
// Tensor-core path: mma.sync m16n8k16 with fp32 accumulation on register fragments.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "oslo_kernels.h"
#include "ptx.cuh"

namespace oslo {

constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

template <typename T> struct Mma;
template <> struct Mma<__nv_bfloat16> {
  static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float x, float y) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Mma<__half> {
  static __device__ __forceinline__ void run(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ uint32_t pack(float x, float y) {
    __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_f(float v) { return __float2half_rn(v); }
};

__device__ __forceinline__ uint32_t s_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // size 0 zero-fills the 16 destination bytes
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct AttnParams {
  const void *q, *k, *v, *o, *dout;
  void *out, *dq, *dk, *dv;
  float* lse;          // [B, H, Sq] natural-log sum-exp of the scaled scores
  const float* delta;  // [B, H, Sq] rowsum(dO * O)
  const uint8_t* kpm;  // [B, Sk] 1 = keep, or nullptr
  int B, H, Sq, Sk;
  long long q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss, do_sb, do_sh, do_ss;
  float scale;
  int causal, window;
};

constexpr int ATT_THREADS = 128;

// copy ROWS x D elements (row stride `stride` in global) into a padded shared tile; rows >= valid are zeroed
template <typename T, int D, int ROWS>
__device__ __forceinline__ void load_tile(T* sm, const T* g, long long stride, int row0, int valid_rows) {
  constexpr int PITCH = D + 8;
  constexpr int CPR = D / 8;  // 16-byte chunks per row
  for (int i = threadIdx.x; i < ROWS * CPR; i += ATT_THREADS) {
    const int r = i / CPR, c = i % CPR;
    const bool ok = (row0 + r) < valid_rows;
    const T* src = g + static_cast<long long>(ok ? row0 + r : 0) * stride + c * 8;
    cp_async16(s_addr(sm + r * PITCH + c * 8), src, ok);
  }
}

__device__ __forceinline__ bool key_visible(int qrow, int kcol, int offset, int Sk, int causal, int window,
                                            const uint8_t* kpm_row) {
  if (kcol >= Sk) return false;
  const int qpos = qrow + offset;
  if (causal && kcol > qpos) return false;
  if (window > 0 && kcol <= qpos - window) return false;
  if (kpm_row && !kpm_row[kcol]) return false;
  return true;
}

// C[16 x (8*NT)] += A[16 x D] (rows a_row0.. of tile As) * B^T where B rows are rows b_row0.. of tile Bs
template <typename T, int D, int NT>
__device__ __forceinline__ void gemm_rowrow(float (&acc)[NT][4], const T* As, int a_row0, const T* Bs, int b_row0) {
  constexpr int PITCH = D + 8;
  const int l = threadIdx.x & 31;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    ldsm_x4(a, s_addr(As + (a_row0 + (l & 7) + ((l >> 3) & 1) * 8) * PITCH + kk * 16 + (l >> 4) * 8));
#pragma unroll
    for (int nt = 0; nt < NT; nt += 2) {
      uint32_t b[4];
      ldsm_x4(b, s_addr(Bs + (b_row0 + nt * 8 + (l & 7) + (l >> 4) * 8) * PITCH + kk * 16 + ((l >> 3) & 1) * 8));
      Mma<T>::run(acc[nt], a, b[0], b[1]);
      Mma<T>::run(acc[nt + 1], a, b[2], b[3]);
    }
  }
}

// O[16 x D] += P[16 x (8*NT)] (register fragments) * V where V rows are rows v_row0.. of tile Vs ([rows][D])
template <typename T, int D, int NT>
__device__ __forceinline__ void gemm_pv(float (&o)[D / 8][4], const uint32_t (&pf)[NT / 2][4], const T* Vs,
                                        int v_row0) {
  constexpr int PITCH = D + 8;
  const int l = threadIdx.x & 31;
#pragma unroll
  for (int ks = 0; ks < NT / 2; ++ks) {
#pragma unroll
    for (int dt = 0; dt < D / 8; dt += 2) {
      uint32_t b[4];
      ldsm_x4_t(b, s_addr(Vs + (v_row0 + ks * 16 + (l & 7) + ((l >> 3) & 1) * 8) * PITCH + dt * 8 + (l >> 4) * 8));
      Mma<T>::run(o[dt], pf[ks], b[0], b[1]);
      Mma<T>::run(o[dt + 1], pf[ks], b[2], b[3]);
    }
  }
}

template <typename T, int NT>
__device__ __forceinline__ void to_afrag(uint32_t (&pf)[NT / 2][4], const float (&s)[NT][4]) {
#pragma unroll
  for (int ks = 0; ks < NT / 2; ++ks) {
    pf[ks][0] = Mma<T>::pack(s[2 * ks][0], s[2 * ks][1]);
    pf[ks][1] = Mma<T>::pack(s[2 * ks][2], s[2 * ks][3]);
    pf[ks][2] = Mma<T>::pack(s[2 * ks + 1][0], s[2 * ks + 1][1]);
    pf[ks][3] = Mma<T>::pack(s[2 * ks + 1][2], s[2 * ks + 1][3]);
  }
}

// ---------------------------------------------------------------------- forward
template <typename T, int D>
__global__ void __launch_bounds__(ATT_THREADS) flash_fwd_kernel(const AttnParams p) {
  constexpr int BM = 64, BN = 64, NT = BN / 8, PITCH = D + 8;
  extern __shared__ __align__(16) uint8_t smem_att[];
  T* Qs = reinterpret_cast<T*>(smem_att);
  T* Ks = Qs + BM * PITCH;
  T* Vs = Ks + BN * PITCH;
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BM;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const T* qg = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
  const T* kg = reinterpret_cast<const T*>(p.k) + b * p.k_sb + h * p.k_sh;
  const T* vg = reinterpret_cast<const T*>(p.v) + b * p.v_sb + h * p.v_sh;
  const uint8_t* kpm_row = p.kpm ? p.kpm + static_cast<long long>(b) * p.Sk : nullptr;
  const int offset = p.Sk - p.Sq;
  int key_hi = p.Sk, key_lo = 0;
  if (p.causal) key_hi = min(p.Sk, q0 + BM + offset);
  if (p.window > 0) key_lo = max(0, q0 + offset - p.window + 1) / BN * BN;
  key_hi = max(key_hi, 0);

  load_tile<T, D, BM>(Qs, qg, p.q_ss, q0, p.Sq);
  if (key_lo < key_hi) load_tile<T, D, BN>(Ks, kg, p.k_ss, key_lo, p.Sk);
  cp_commit();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
  float mrow[2] = {-CUDART_INF_F, -CUDART_INF_F}, lrow[2] = {0.f, 0.f};
  const float sc = p.scale * LOG2E;
  const int r0 = q0 + w * 16 + (l >> 2);  // this thread's rows: r0 and r0 + 8

  for (int n0 = key_lo; n0 < key_hi; n0 += BN) {
    cp_wait<0>();
    __syncthreads();
    load_tile<T, D, BN>(Vs, vg, p.v_ss, n0, p.Sk);
    cp_commit();
    float s[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
    gemm_rowrow<T, D, NT>(s, Qs, w * 16, Ks, 0);
    float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = r0 + (e >> 1) * 8;
        const int col = n0 + nt * 8 + (l & 3) * 2 + (e & 1);
        const bool vis = key_visible(row, col, offset, p.Sk, p.causal, p.window, kpm_row);
        s[nt][e] = vis ? s[nt][e] * sc : -CUDART_INF_F;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
      }
    }
    float alpha[2], msafe[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      const float mn = fmaxf(mrow[i], mx[i]);
      msafe[i] = (mn == -CUDART_INF_F) ? 0.f : mn;
      alpha[i] = exp2f(mrow[i] - msafe[i]);  // exp2(-inf) = 0 on the first block
      mrow[i] = mn;
      lrow[i] *= alpha[i];
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = exp2f(s[nt][e] - msafe[e >> 1]);
        s[nt][e] = pv;
        lrow[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= alpha[0]; o[i][1] *= alpha[0]; o[i][2] *= alpha[1]; o[i][3] *= alpha[1];
    }
    uint32_t pf[NT / 2][4];
    to_afrag<T, NT>(pf, s);
    cp_wait<0>();
    __syncthreads();
    if (n0 + BN < key_hi) load_tile<T, D, BN>(Ks, kg, p.k_ss, n0 + BN, p.Sk);
    cp_commit();
    gemm_pv<T, D, NT>(o, pf, Vs, 0);
  }
  cp_wait<0>();

  T* og = reinterpret_cast<T*>(p.out) + b * p.o_sb + h * p.o_sh;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 1);
    lrow[i] += __shfl_xor_sync(0xffffffffu, lrow[i], 2);
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + i * 8;
    if (row >= p.Sq) continue;
    const float inv = lrow[i] > 0.f ? 1.f / lrow[i] : 0.f;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      const uint32_t packed = Mma<T>::pack(o[dt][2 * i] * inv, o[dt][2 * i + 1] * inv);
      *reinterpret_cast<uint32_t*>(og + static_cast<long long>(row) * p.o_ss + dt * 8 + (l & 3) * 2) = packed;
    }
    if ((l & 3) == 0 && p.lse) {
      const float lse = lrow[i] > 0.f ? (mrow[i] + log2f(lrow[i])) * LN2 : 0.f;
      p.lse[(static_cast<long long>(b) * p.H + h) * p.Sq + row] = lse;
    }
  }
}

// ---------------------------------------------------------------------- backward: delta = rowsum(dO * O)
template <typename T>
__global__ void attn_delta_kernel(const AttnParams p, float* delta, int D) {
  const long long row = blockIdx.x * static_cast<long long>(blockDim.x / 32) + (threadIdx.x >> 5);
  const long long total = static_cast<long long>(p.B) * p.H * p.Sq;
  if (row >= total) return;
  const int l = threadIdx.x & 31;
  const int s = static_cast<int>(row % p.Sq);
  const int h = static_cast<int>((row / p.Sq) % p.H);
  const int b = static_cast<int>(row / (static_cast<long long>(p.Sq) * p.H));
  const T* o = reinterpret_cast<const T*>(p.o) + b * p.o_sb + h * p.o_sh + static_cast<long long>(s) * p.o_ss;
  const T* g = reinterpret_cast<const T*>(p.dout) + b * p.do_sb + h * p.do_sh + static_cast<long long>(s) * p.do_ss;
  float acc = 0.f;
  for (int d = l; d < D; d += 32) acc += Mma<T>::to_f(o[d]) * Mma<T>::to_f(g[d]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (l == 0) delta[row] = acc;
}

// ---------------------------------------------------------------------- backward: dQ pass
template <typename T, int D>
__global__ void __launch_bounds__(ATT_THREADS) flash_bwd_dq_kernel(const AttnParams p) {
  constexpr int BM = 64, BN = 32, NT = BN / 8, PITCH = D + 8;
  extern __shared__ __align__(16) uint8_t smem_att[];
  T* Qs = reinterpret_cast<T*>(smem_att);
  T* Gs = Qs + BM * PITCH;  // dO
  T* Ks = Gs + BM * PITCH;
  T* Vs = Ks + BN * PITCH;
  const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * BM;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const T* qg = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
  const T* kg = reinterpret_cast<const T*>(p.k) + b * p.k_sb + h * p.k_sh;
  const T* vg = reinterpret_cast<const T*>(p.v) + b * p.v_sb + h * p.v_sh;
  const T* gg = reinterpret_cast<const T*>(p.dout) + b * p.do_sb + h * p.do_sh;
  const uint8_t* kpm_row = p.kpm ? p.kpm + static_cast<long long>(b) * p.Sk : nullptr;
  const int offset = p.Sk - p.Sq;
  int key_hi = p.Sk, key_lo = 0;
  if (p.causal) key_hi = max(0, min(p.Sk, q0 + BM + offset));
  if (p.window > 0) key_lo = max(0, q0 + offset - p.window + 1) / BN * BN;

  load_tile<T, D, BM>(Qs, qg, p.q_ss, q0, p.Sq);
  load_tile<T, D, BM>(Gs, gg, p.do_ss, q0, p.Sq);
  cp_commit();

  const float sc = p.scale * LOG2E;
  const int r0 = q0 + w * 16 + (l >> 2);
  float lse2[2], dl[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + i * 8;
    const long long idx = (static_cast<long long>(b) * p.H + h) * p.Sq + row;
    lse2[i] = row < p.Sq ? p.lse[idx] * LOG2E : 0.f;
    dl[i] = row < p.Sq ? p.delta[idx] : 0.f;
  }
  float dq[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f; }

  for (int n0 = key_lo; n0 < key_hi; n0 += BN) {
    __syncthreads();  // previous iteration finished reading Ks / Vs
    load_tile<T, D, BN>(Ks, kg, p.k_ss, n0, p.Sk);
    load_tile<T, D, BN>(Vs, vg, p.v_ss, n0, p.Sk);
    cp_commit();
    cp_wait<0>();
    __syncthreads();
    float s[NT][4], dp[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
    }
    gemm_rowrow<T, D, NT>(s, Qs, w * 16, Ks, 0);
    gemm_rowrow<T, D, NT>(dp, Gs, w * 16, Vs, 0);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int row = r0 + (e >> 1) * 8;
        const int col = n0 + nt * 8 + (l & 3) * 2 + (e & 1);
        const bool vis = row < p.Sq && key_visible(row, col, offset, p.Sk, p.causal, p.window, kpm_row);
        const float pr = vis ? exp2f(s[nt][e] * sc - lse2[e >> 1]) : 0.f;
        s[nt][e] = pr * (dp[nt][e] - dl[e >> 1]) * p.scale;  // dS
      }
    }
    uint32_t df[NT / 2][4];
    to_afrag<T, NT>(df, s);
    gemm_pv<T, D, NT>(dq, df, Ks, 0);
  }
  T* dg = reinterpret_cast<T*>(p.dq) + b * p.q_sb + h * p.q_sh;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = r0 + i * 8;
    if (row >= p.Sq) continue;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      *reinterpret_cast<uint32_t*>(dg + static_cast<long long>(row) * p.q_ss + dt * 8 + (l & 3) * 2) =
          Mma<T>::pack(dq[dt][2 * i], dq[dt][2 * i + 1]);
    }
  }
}

// ---------------------------------------------------------------------- backward: dK / dV pass
// Transposed orientation: rows = keys (16 per warp, 64 per CTA), columns = queries (blocks of 32).
template <typename T, int D, bool DO_DK, bool DO_DV>
__global__ void __launch_bounds__(ATT_THREADS) flash_bwd_dkv_kernel(const AttnParams p) {
  constexpr int BN = 64, BQ = 32, NT = BQ / 8, PITCH = D + 8;
  extern __shared__ __align__(16) uint8_t smem_att[];
  T* Ks = reinterpret_cast<T*>(smem_att);
  T* Vs = Ks + BN * PITCH;
  T* Qs = Vs + BN * PITCH;
  T* Gs = Qs + BQ * PITCH;
  float* lse_s = reinterpret_cast<float*>(Gs + BQ * PITCH);
  float* dl_s = lse_s + BQ;
  const int b = blockIdx.z, h = blockIdx.y, k0 = blockIdx.x * BN;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const T* qg = reinterpret_cast<const T*>(p.q) + b * p.q_sb + h * p.q_sh;
  const T* kg = reinterpret_cast<const T*>(p.k) + b * p.k_sb + h * p.k_sh;
  const T* vg = reinterpret_cast<const T*>(p.v) + b * p.v_sb + h * p.v_sh;
  const T* gg = reinterpret_cast<const T*>(p.dout) + b * p.do_sb + h * p.do_sh;
  const uint8_t* kpm_row = p.kpm ? p.kpm + static_cast<long long>(b) * p.Sk : nullptr;
  const int offset = p.Sk - p.Sq;
  // queries that can see keys [k0, k0 + BN): q + offset >= k0 (causal), q + offset - window < k0 + BN - 1 + 1
  int q_lo = 0, q_hi = p.Sq;
  if (p.causal) q_lo = max(0, k0 - offset) / BQ * BQ;
  if (p.window > 0) q_hi = min(p.Sq, k0 + BN - 1 - offset + p.window);
  q_hi = max(q_hi, 0);

  load_tile<T, D, BN>(Ks, kg, p.k_ss, k0, p.Sk);
  load_tile<T, D, BN>(Vs, vg, p.v_ss, k0, p.Sk);
  cp_commit();

  const float sc = p.scale * LOG2E;
  const int kr0 = k0 + w * 16 + (l >> 2);  // this thread's key rows: kr0, kr0 + 8
  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
  }
  const long long stat_base = (static_cast<long long>(b) * p.H + h) * p.Sq;

  for (int m0 = q_lo; m0 < q_hi; m0 += BQ) {
    __syncthreads();
    load_tile<T, D, BQ>(Qs, qg, p.q_ss, m0, p.Sq);
    load_tile<T, D, BQ>(Gs, gg, p.do_ss, m0, p.Sq);
    cp_commit();
    if (threadIdx.x < BQ) {
      const int row = m0 + threadIdx.x;
      lse_s[threadIdx.x] = row < p.Sq ? p.lse[stat_base + row] * LOG2E : 0.f;
      dl_s[threadIdx.x] = row < p.Sq ? p.delta[stat_base + row] : 0.f;
    }
    cp_wait<0>();
    __syncthreads();
    float st[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) { st[i][0] = st[i][1] = st[i][2] = st[i][3] = 0.f; }
    gemm_rowrow<T, D, NT>(st, Ks, w * 16, Qs, 0);  // S^T = K Q^T
    float dpt[NT][4];
    if (DO_DK) {
#pragma unroll
      for (int i = 0; i < NT; ++i) { dpt[i][0] = dpt[i][1] = dpt[i][2] = dpt[i][3] = 0.f; }
      gemm_rowrow<T, D, NT>(dpt, Vs, w * 16, Gs, 0);  // dP^T = V dO^T
    }
    float ds[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = kr0 + (e >> 1) * 8;
        const int ql = nt * 8 + (l & 3) * 2 + (e & 1);
        const int qrow = m0 + ql;
        const bool vis = qrow < p.Sq && key_visible(qrow, key, offset, p.Sk, p.causal, p.window, kpm_row);
        const float pr = vis ? exp2f(st[nt][e] * sc - lse_s[ql]) : 0.f;
        st[nt][e] = pr;
        if (DO_DK) ds[nt][e] = pr * (dpt[nt][e] - dl_s[ql]) * p.scale;
      }
    }
    if (DO_DV) {
      uint32_t pf[NT / 2][4];
      to_afrag<T, NT>(pf, st);
      gemm_pv<T, D, NT>(dv, pf, Gs, 0);  // dV += P^T dO
    }
    if (DO_DK) {
      uint32_t df[NT / 2][4];
      to_afrag<T, NT>(df, ds);
      gemm_pv<T, D, NT>(dk, df, Qs, 0);  // dK += dS^T Q
    }
  }
  cp_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int key = kr0 + i * 8;
    if (key >= p.Sk) continue;
    if (DO_DK) {
      T* dg = reinterpret_cast<T*>(p.dk) + b * p.k_sb + h * p.k_sh + static_cast<long long>(key) * p.k_ss;
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt)
        *reinterpret_cast<uint32_t*>(dg + dt * 8 + (l & 3) * 2) = Mma<T>::pack(dk[dt][2 * i], dk[dt][2 * i + 1]);
    }
    if (DO_DV) {
      T* dg = reinterpret_cast<T*>(p.dv) + b * p.v_sb + h * p.v_sh + static_cast<long long>(key) * p.v_ss;
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt)
        *reinterpret_cast<uint32_t*>(dg + dt * 8 + (l & 3) * 2) = Mma<T>::pack(dv[dt][2 * i], dv[dt][2 * i + 1]);
    }
  }
}

// ---------------------------------------------------------------------- decode attention (one query per row)
// grid (splits, H, B); each CTA scans a slice of the cache with online softmax and writes a partial
// (max, sum, out[D]) to the workspace; the combine kernel merges the slices.
template <typename T>
__global__ void __launch_bounds__(128) decode_attn_kernel(const T* __restrict__ q, const T* __restrict__ kc,
                                                          const T* __restrict__ vc, const int* __restrict__ lengths,
                                                          float* __restrict__ ws, int H, int Tmax, int D, int splits,
                                                          float scale, int window, int* err) {
  extern __shared__ float sm_dec[];
  float* qs = sm_dec;             // [D]
  float* red = qs + D;            // [4][D] per-warp partial outputs
  float* stat = red + 4 * D;      // [4][2]
  const int b = blockIdx.z, h = blockIdx.y, sp = blockIdx.x;
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  int len = lengths[b];
  if (len < 0 || len > Tmax) {   // a length that does not fit the cache: never read past it
    OSLO_REPORT_BOUNDS(err);
    len = len < 0 ? 0 : Tmax;
  }
  int lo = 0;
  if (window > 0) lo = max(0, len - window);
  const int span = len - lo;
  const int per = (span + splits - 1) / splits;
  const int t0 = lo + sp * per, t1 = min(len, t0 + per);
  const T* qp = q + (static_cast<long long>(b) * H + h) * D;
  for (int d = threadIdx.x; d < D; d += 128) qs[d] = Mma<T>::to_f(qp[d]) * scale * LOG2E;
  __syncthreads();
  const T* kb = kc + (static_cast<long long>(b) * H + h) * Tmax * D;
  const T* vb = vc + (static_cast<long long>(b) * H + h) * Tmax * D;
  float m = -CUDART_INF_F, s = 0.f;
  float acc[8];  // lane owns dims l*8.. (D <= 256) in 16-byte chunks
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  const bool lane_active = l * 8 < D;
  // each warp walks its keys in batches of KB: all K and V rows of a batch are requested before any of them is
  // used, so a warp keeps 2 * KB 16-byte loads in flight instead of one (the scan is latency-bound otherwise)
  constexpr int KB = 8;
  for (int tb = t0 + w * KB; tb < t1; tb += 4 * KB) {
    uint4 kraw[KB], vraw[KB];
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      const int t = tb + j;
      if (lane_active && t < t1) {
        kraw[j] = *reinterpret_cast<const uint4*>(kb + static_cast<long long>(t) * D + l * 8);
        vraw[j] = *reinterpret_cast<const uint4*>(vb + static_cast<long long>(t) * D + l * 8);
      } else {
        kraw[j] = make_uint4(0, 0, 0, 0);
        vraw[j] = make_uint4(0, 0, 0, 0);
      }
    }
    float dot[KB];
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      const T* e = reinterpret_cast<const T*>(&kraw[j]);
      float d = 0.f;
      if (lane_active) {
#pragma unroll
        for (int i = 0; i < 8; ++i) d += Mma<T>::to_f(e[i]) * qs[l * 8 + i];
      }
      dot[j] = d;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
      for (int j = 0; j < KB; ++j) dot[j] += __shfl_xor_sync(0xffffffffu, dot[j], off);
    }
    float mn = m;
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      if (tb + j >= t1) dot[j] = -CUDART_INF_F;
      mn = fmaxf(mn, dot[j]);
    }
    const float a = exp2f(m - mn);   // m = -inf on the first batch: a = 0 and s, acc are 0 anyway
    float ps = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= a;
#pragma unroll
    for (int j = 0; j < KB; ++j) {
      const float pr = exp2f(dot[j] - mn);
      ps += pr;
      const T* e = reinterpret_cast<const T*>(&vraw[j]);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += pr * Mma<T>::to_f(e[i]);
    }
    s = s * a + ps;
    m = mn;
  }
  if (l == 0) { stat[w * 2] = m; stat[w * 2 + 1] = s; }
  __syncthreads();
  float gm = fmaxf(fmaxf(stat[0], stat[2]), fmaxf(stat[4], stat[6]));
  const float mine = (m == -CUDART_INF_F) ? 0.f : exp2f(m - gm);
  if (lane_active) {
#pragma unroll
    for (int i = 0; i < 8; ++i) red[w * D + l * 8 + i] = acc[i] * mine;
  }
  __syncthreads();
  float gs = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) gs += (stat[i * 2] == -CUDART_INF_F) ? 0.f : stat[i * 2 + 1] * exp2f(stat[i * 2] - gm);
  float* out = ws + ((static_cast<long long>(b) * H + h) * splits + sp) * (D + 2);
  for (int d = threadIdx.x; d < D; d += 128) out[d] = red[d] + red[D + d] + red[2 * D + d] + red[3 * D + d];
  if (threadIdx.x == 0) { out[D] = gm; out[D + 1] = gs; }
}
template <typename T>
__global__ void decode_combine_kernel(const float* __restrict__ ws, T* __restrict__ o, int D, int splits) {
  const long long bh = blockIdx.x;
  const float* base = ws + bh * splits * (D + 2);
  float gm = -CUDART_INF_F;
  for (int s = 0; s < splits; ++s) gm = fmaxf(gm, base[s * (D + 2) + D]);
  float tot = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = base[s * (D + 2) + D];
    if (m != -CUDART_INF_F) tot += base[s * (D + 2) + D + 1] * exp2f(m - gm);
  }
  const float inv = tot > 0.f ? 1.f / tot : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float m = base[s * (D + 2) + D];
      if (m != -CUDART_INF_F) a += base[s * (D + 2) + d] * exp2f(m - gm);
    }
    o[bh * D + d] = Mma<T>::from_f(a * inv);
  }
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  return static_cast<int>(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)));
}

static void fill_params(AttnParams& p, const void* q, const void* k, const void* v, int B, int H, int Sq, int Sk,
                        long long q_sb, long long q_sh, long long q_ss, long long k_sb, long long k_sh,
                        long long k_ss, long long v_sb, long long v_sh, long long v_ss, long long o_sb,
                        long long o_sh, long long o_ss, float scale, int causal, int window, const uint8_t* kpm) {
  p.q = q; p.k = k; p.v = v; p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk;
  p.q_sb = q_sb; p.q_sh = q_sh; p.q_ss = q_ss; p.k_sb = k_sb; p.k_sh = k_sh; p.k_ss = k_ss;
  p.v_sb = v_sb; p.v_sh = v_sh; p.v_ss = v_ss; p.o_sb = o_sb; p.o_sh = o_sh; p.o_ss = o_ss;
  p.scale = scale; p.causal = causal; p.window = window; p.kpm = kpm;
  p.o = nullptr; p.dout = nullptr; p.out = nullptr; p.dq = p.dk = p.dv = nullptr; p.lse = nullptr; p.delta = nullptr;
  p.do_sb = p.do_sh = p.do_ss = 0;
}

template <typename T, int D>
static int launch_fwd(const AttnParams& p, cudaStream_t st) {
  constexpr size_t smem = 3 * 64 * (D + 8) * sizeof(T);
  int rc = set_smem(flash_fwd_kernel<T, D>, smem);
  if (rc) return rc;
  dim3 grid((p.Sq + 63) / 64, p.H, p.B);
  flash_fwd_kernel<T, D><<<grid, ATT_THREADS, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

template <typename T, int D>
static int launch_bwd(const AttnParams& p, float* delta, cudaStream_t st) {
  const long long rows = static_cast<long long>(p.B) * p.H * p.Sq;
  attn_delta_kernel<T><<<static_cast<unsigned>((rows + 3) / 4), 128, 0, st>>>(p, delta, D);
  {
    constexpr size_t smem = (2 * 64 + 2 * 32) * (D + 8) * sizeof(T);
    int rc = set_smem(flash_bwd_dq_kernel<T, D>, smem);
    if (rc) return rc;
    dim3 grid((p.Sq + 63) / 64, p.H, p.B);
    flash_bwd_dq_kernel<T, D><<<grid, ATT_THREADS, smem, st>>>(p);
  }
  {
    constexpr size_t smem = (2 * 64 + 2 * 32) * (D + 8) * sizeof(T) + 2 * 32 * sizeof(float);
    dim3 grid((p.Sk + 63) / 64, p.H, p.B);
    if constexpr (D <= 128) {
      int rc = set_smem(flash_bwd_dkv_kernel<T, D, true, true>, smem);
      if (rc) return rc;
      flash_bwd_dkv_kernel<T, D, true, true><<<grid, ATT_THREADS, smem, st>>>(p);
    } else {  // 2 x [16 x 256] fp32 accumulators do not fit the register file: one pass per gradient
      int rc = set_smem(flash_bwd_dkv_kernel<T, D, true, false>, smem);
      if (rc) return rc;
      rc = set_smem(flash_bwd_dkv_kernel<T, D, false, true>, smem);
      if (rc) return rc;
      flash_bwd_dkv_kernel<T, D, true, false><<<grid, ATT_THREADS, smem, st>>>(p);
      flash_bwd_dkv_kernel<T, D, false, true><<<grid, ATT_THREADS, smem, st>>>(p);
    }
  }
  return static_cast<int>(cudaGetLastError());
}

}  // namespace oslo

using namespace oslo;

#define ATT_DISPATCH(dtype, D, ...)                                                      \
  if (dtype == OSLO_DT_BF16) {                                                           \
    using T = __nv_bfloat16;                                                             \
    if (D == 64) { constexpr int HD = 64; __VA_ARGS__ } else if (D == 128) { constexpr int HD = 128; __VA_ARGS__ } \
    else if (D == 256) { constexpr int HD = 256; __VA_ARGS__ } else return -3;                  \
  } else if (dtype == OSLO_DT_FP16) {                                                    \
    using T = __half;                                                                    \
    if (D == 64) { constexpr int HD = 64; __VA_ARGS__ } else if (D == 128) { constexpr int HD = 128; __VA_ARGS__ } \
    else if (D == 256) { constexpr int HD = 256; __VA_ARGS__ } else return -3;                  \
  } else return -2;

extern "C" int oslo_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const uint8_t* kpm,
                              int B, int H, int Sq, int Sk, int D, long long q_sb, long long q_sh, long long q_ss,
                              long long k_sb, long long k_sh, long long k_ss, long long v_sb, long long v_sh,
                              long long v_ss, long long o_sb, long long o_sh, long long o_ss, float scale, int causal,
                              int window, int dtype, cudaStream_t st) {
  if (B * H * Sq == 0) return 0;
  AttnParams p;
  fill_params(p, q, k, v, B, H, Sq, Sk, q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss,
              scale, causal, window, kpm);
  p.out = o; p.lse = lse;
  ATT_DISPATCH(dtype, D, { return launch_fwd<T, HD>(p, st); })
}

extern "C" int oslo_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                              const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv,
                              const uint8_t* kpm, int B, int H, int Sq, int Sk, int D, long long q_sb, long long q_sh,
                              long long q_ss, long long k_sb, long long k_sh, long long k_ss, long long v_sb,
                              long long v_sh, long long v_ss, long long o_sb, long long o_sh, long long o_ss,
                              long long do_sb, long long do_sh, long long do_ss, float scale, int causal, int window,
                              int dtype, cudaStream_t st) {
  (void)dq_acc;
  if (B * H * Sq == 0) return 0;
  AttnParams p;
  fill_params(p, q, k, v, B, H, Sq, Sk, q_sb, q_sh, q_ss, k_sb, k_sh, k_ss, v_sb, v_sh, v_ss, o_sb, o_sh, o_ss,
              scale, causal, window, kpm);
  p.o = o; p.dout = dout; p.lse = const_cast<float*>(lse); p.delta = delta;
  p.dq = dq; p.dk = dk; p.dv = dv; p.do_sb = do_sb; p.do_sh = do_sh; p.do_ss = do_ss;
  ATT_DISPATCH(dtype, D, { return launch_bwd<T, HD>(p, delta, st); })
}

extern "C" int oslo_decode_attn(const void* q, const void* kc, const void* vc, void* o, const int* lengths, float* ws,
                                int B, int H, int T, int D, int splits, float scale, int window, int dtype,
                                int* err_word, cudaStream_t st) {
  if (B * H == 0) return 0;
  if (D % 8 || D > 256) return -3;
  const size_t smem = (D + 4 * D + 8) * sizeof(float);
  dim3 grid(splits, H, B);
  if (dtype == OSLO_DT_BF16) {
    decode_attn_kernel<__nv_bfloat16><<<grid, 128, smem, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)kc,
                                                               (const __nv_bfloat16*)vc, lengths, ws, H, T, D, splits,
                                                               scale, window, err_word);
    decode_combine_kernel<__nv_bfloat16><<<B * H, 128, 0, st>>>(ws, (__nv_bfloat16*)o, D, splits);
  } else if (dtype == OSLO_DT_FP16) {
    decode_attn_kernel<__half><<<grid, 128, smem, st>>>((const __half*)q, (const __half*)kc, (const __half*)vc, lengths,
                                                        ws, H, T, D, splits, scale, window, err_word);
    decode_combine_kernel<__half><<<B * H, 128, 0, st>>>(ws, (__half*)o, D, splits);
  } else {
    return -2;
  }
  return static_cast<int>(cudaGetLastError());
}
