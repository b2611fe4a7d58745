// Flash attention backward on the tcgen05 tensor cores with TMEM accumulators.
//
// Three launches of one kernel template, each a "resident rows x streamed column blocks" pipeline in which one
// TMEM lane (and one transform thread) owns one resident row:
//
//   dV  rows = 128 keys     S^T = K Q^T                 P^T = exp2(S^T - lse[q])              dV += P^T dO
//   dK  rows = 128 keys     S^T = K Q^T, dP^T = V dO^T  dS^T = P^T o (dP^T - delta[q])        dK += dS^T Q
//   dQ  rows = 128 queries  S = Q K^T,   dP = dO V^T    dS = P o (dP - delta[q])              dQ += dS K
//
// The first-stage products land in double-buffered TMEM columns; the transform warps read them with tcgen05.ld,
// write the 16-bit P / dS tile back into the same TMEM columns (two elements per 32-bit column) and the second
// stage reads it from tensor memory as its A operand. The streamed operand of the second stage is the same
// shared-memory tile the first stage used as a K-major operand, now described as MN-major, so nothing is
// transposed or copied. Softmax statistics that belong to columns (dV, dK) are staged in shared memory by the
// otherwise idle lanes of the producer warp. Head dim 256 splits into three launches because the two [128 x 256]
// fp32 accumulators of dK and dV plus the S / dP buffers exceed the 512 TMEM columns of an SM.
//
// 192 threads: warp 0 = TMA producer (+ statistics), warp 1 = TMEM owner and MMA issuer, warps 2-5 = transform and
// epilogue. Every wait is bounded (ptx.cuh).
//
// Reference behaviour covered: the backward of the same path - softmax backward kernels of
// oslo/fused_kernels/includes/fused_triang_softmax.h:253-351 / fused_softmax.h:224-325 around autograd's batched
// matmuls - without ever materialising the [S, S] probabilities.
#include "attention_sm100.cuh"

namespace oslo {

enum : int { BWD_DV = 0, BWD_DK = 1, BWD_DQ = 2 };

struct FaBwdParams {
  void* out;            // gradient written by this launch; its rows are the resident rows
  long long o_sb, o_sh, o_ss;
  const float* lse;     // [B, H, Sq] natural-log sum-exp of the scaled scores
  const float* delta;   // [B, H, Sq] rowsum(dO o O)
  const uint8_t* kpm;   // [B, Sk] 1 = keep, or nullptr
  int B, H, Sq, Sk;
  float scale;
  int causal, window, fp16;
  // where (seq, head, batch) sit in the tensor maps of the resident operands r1, r2 and the streamed s1, s2
  int r1_pos[3], r2_pos[3], s1_pos[3], s2_pos[3];
  int* err;
};

// delta[b, h, q] = sum_d dO[b, h, q, d] * O[b, h, q, d]; one warp per row
template <typename T>
__global__ void fa_delta_kernel(const T* __restrict__ o, const T* __restrict__ dout, float* __restrict__ delta, int B,
                                int H, int Sq, int D, long long o_sb, long long o_sh, long long o_ss, long long d_sb,
                                long long d_sh, long long d_ss) {
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= static_cast<long long>(B) * H * Sq) return;
  const int q = static_cast<int>(row % Sq);
  const int h = static_cast<int>((row / Sq) % H);
  const int b = static_cast<int>(row / (static_cast<long long>(Sq) * H));
  const T* op = o + b * o_sb + h * o_sh + q * o_ss;
  const T* dp = dout + b * d_sb + h * d_sh + q * d_ss;
  float acc = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const uint32_t a = *reinterpret_cast<const uint32_t*>(op + d);
    const uint32_t g = *reinterpret_cast<const uint32_t*>(dp + d);
    float a0, a1, g0, g1;
    if (sizeof(T) == 2 && std::is_same<T, __half>::value) {
      const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&a));
      const float2 fg = __half22float2(*reinterpret_cast<const __half2*>(&g));
      a0 = fa.x; a1 = fa.y; g0 = fg.x; g1 = fg.y;
    } else {
      const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a));
      const float2 fg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g));
      a0 = fa.x; a1 = fa.y; g0 = fg.x; g1 = fg.y;
    }
    acc += a0 * g0 + a1 * g1;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[row] = acc;
}

__device__ __forceinline__ bool fa_visible(int q, int k, int offset, int Sq, int Sk, int causal, int window) {
  if (k >= Sk || q >= Sq) return false;
  const int qpos = q + offset;
  if (causal && k > qpos) return false;
  if (window > 0 && k <= qpos - window) return false;
  return true;
}

// D = head dim, BN = streamed block (columns of the first-stage tiles), S1N / S2N = ring depths of the two
// streamed operands. Streamed operand s1 feeds S (or S^T); s2 feeds dP (dK, dQ) or the second stage (dV).
template <int D, int BN, int MODE, int S1N, int S2N>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tr1, const __grid_constant__ CUtensorMap tr2,
              const __grid_constant__ CUtensorMap ts1, const __grid_constant__ CUtensorMap ts2, const FaBwdParams p) {
  constexpr bool TWO = MODE != BWD_DV;            // two first-stage products, two resident operands
  constexpr bool KEY_ROWS = MODE != BWD_DQ;       // resident rows are keys, streamed columns are queries
  constexpr int DC = D / 64;
  constexpr uint32_t R_SUB = FA_BM * 128;         // one [128 x 64] sub-tile
  constexpr uint32_t S_SUB = BN * 128;            // one [BN x 64] sub-tile
  constexpr uint32_t R_BYTES = DC * R_SUB;
  constexpr uint32_t S_BYTES = DC * S_SUB;
  constexpr uint32_t NRES = TWO ? 2 : 1;
  constexpr uint32_t STAT_BYTES = KEY_ROWS ? 2 * 2 * BN * 4 : 0;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t DP_COL = 2 * BN;             // S buffers at 0 and BN; dP buffers (TWO) at 2 BN and 3 BN
  constexpr uint32_t ACC_COL = TWO ? 4 * BN : 2 * BN;
  static_assert(ACC_COL + D <= TMEM_COLS, "TMEM budget");
  constexpr int B_RFULL = 0, B_S1F = 1, B_S1E = B_S1F + S1N, B_S2F = B_S1E + S1N, B_S2E = B_S2F + S2N,
                B_SPF = B_S2E + S2N, B_TRD = B_SPF + 2, B_STF = B_TRD + 2, B_ACC = B_STF + 2, NBAR = B_ACC + 1;

  extern __shared__ uint8_t fa_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t r1_s = smem_u32(smem);
  const uint32_t r2_s = r1_s + R_BYTES;           // only when TWO
  const uint32_t s1_s = r1_s + NRES * R_BYTES;
  const uint32_t s2_s = s1_s + S1N * S_BYTES;
  constexpr uint32_t TILE_BYTES = NRES * R_BYTES + (S1N + S2N) * S_BYTES;
  float* stats = reinterpret_cast<float*>(smem + TILE_BYTES);   // [2 buffers][2: lse2, delta][BN]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TILE_BYTES + STAT_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int offset = p.Sk - p.Sq;
  const int n_rows = KEY_ROWS ? p.Sk : p.Sq;
  const int n_cols = KEY_ROWS ? p.Sq : p.Sk;
  // heavy tiles first: under a causal mask the last query tile sees the most keys, the first key tile the most queries
  const int tile = KEY_ROWS ? static_cast<int>(blockIdx.x) : static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);
  const int row0 = tile * FA_BM;
  int c_lo = 0, c_hi = n_cols;
  if (KEY_ROWS) {
    if (p.causal) c_lo = max(0, row0 - offset) / BN * BN;
    if (p.window > 0) c_hi = min(n_cols, row0 + FA_BM - 1 - offset + p.window);
  } else {
    if (p.causal) c_hi = min(n_cols, row0 + FA_BM + offset);
    if (p.window > 0) c_lo = max(0, row0 + offset - p.window + 1) / BN * BN;
  }
  const int nblk = c_hi > c_lo ? (c_hi - c_lo + BN - 1) / BN : 0;
  const long long stat_base = (static_cast<long long>(b) * p.H + h) * p.Sq;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NBAR; ++i) mbar_init(bar(i), (i >= B_TRD && i < B_TRD + 2) ? 4 : 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (+ column statistics)
    if (nblk > 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tr1); tma_prefetch_desc(&ts1); tma_prefetch_desc(&ts2);
        if (TWO) tma_prefetch_desc(&tr2);
        mbar_expect_tx(bar(B_RFULL), NRES * R_BYTES);
#pragma unroll
        for (int c = 0; c < DC; ++c) tma_load_rows(r1_s + c * R_SUB, &tr1, bar(B_RFULL), c * 64, row0, h, b, p.r1_pos);
        if (TWO) {
#pragma unroll
          for (int c = 0; c < DC; ++c) tma_load_rows(r2_s + c * R_SUB, &tr2, bar(B_RFULL), c * 64, row0, h, b, p.r2_pos);
        }
      }
      int ok = 1;
      for (int j = 0; j < nblk; ++j) {
        const int c0 = c_lo + j * BN;
        const int st1 = j % S1N, st2 = j % S2N;
        const uint32_t ph1 = (j / S1N) & 1, ph2 = (j / S2N) & 1;
        if (lane == 0) {
          auto load_s1 = [&]() -> bool {
            if (!mbar_wait(bar(B_S1E + st1), ph1 ^ 1, abort_flag, p.err, ERR_WAIT_EMPTY)) return false;
            mbar_expect_tx(bar(B_S1F + st1), S_BYTES);
#pragma unroll
            for (int c = 0; c < DC; ++c)
              tma_load_rows(s1_s + st1 * S_BYTES + c * S_SUB, &ts1, bar(B_S1F + st1), c * 64, c0, h, b, p.s1_pos);
            return true;
          };
          auto load_s2 = [&]() -> bool {
            if (!mbar_wait(bar(B_S2E + st2), ph2 ^ 1, abort_flag, p.err, ERR_WAIT_EMPTY)) return false;
            mbar_expect_tx(bar(B_S2F + st2), S_BYTES);
#pragma unroll
            for (int c = 0; c < DC; ++c)
              tma_load_rows(s2_s + st2 * S_BYTES + c * S_SUB, &ts2, bar(B_S2F + st2), c * 64, c0, h, b, p.s2_pos);
            return true;
          };
          // the MMA warp consumes s2 first when it feeds dP, s1 first when s2 belongs to the second stage
          bool good = TWO ? (load_s2() && load_s1()) : (load_s1() && load_s2());
          // the statistics buffer of block j was last read by the transform of block j - 2
          if (KEY_ROWS && good)
            good = mbar_wait(bar(B_TRD + (j & 1)), ((j >> 1) & 1) ^ 1, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY);
          ok = good ? 1 : 0;
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (KEY_ROWS) {
          float* sb = stats + (j & 1) * 2 * BN;
          for (int i = lane; i < BN; i += 32) {
            const int q = c0 + i;
            float l2 = CUDART_INF_F, dl = 0.f;   // out-of-range query column: exp2(s - inf) = 0
            if (q < p.Sq) {
              l2 = p.lse[stat_base + q] * FA_LOG2E;
              dl = TWO ? p.delta[stat_base + q] : 0.f;
            }
            sb[i] = l2;
            sb[BN + i] = dl;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_STF + (j & 1)));
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && nblk > 0) {
      const int fmt = p.fp16 ? 0 : 1;
      const uint32_t idesc_fs = make_idesc_f16(FA_BM, BN, fmt, 0, 0);
      const uint32_t idesc_ss = make_idesc_f16(FA_BM, D, fmt, 0, 1);
      bool ok = mbar_wait(bar(B_RFULL), 0, abort_flag, p.err, ERR_WAIT_FULL);
      auto first_stage = [&](int j) -> bool {
        const int buf = j & 1, st1 = j % S1N, st2 = j % S2N;
        if (TWO) {
          if (!mbar_wait(bar(B_S2F + st2), (j / S2N) & 1, abort_flag, p.err, ERR_WAIT_FULL)) return false;
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t da = make_smem_desc(r2_s + (kk >> 2) * R_SUB + (kk & 3) * 32, 16, 1024);
            const uint64_t db = make_smem_desc(s2_s + st2 * S_BYTES + (kk >> 2) * S_SUB + (kk & 3) * 32, 16, 1024);
            umma_f16(tmem_base + DP_COL + buf * BN, da, db, idesc_fs, kk != 0);
          }
          umma_commit(bar(B_S2E + st2));
        }
        if (!mbar_wait(bar(B_S1F + st1), (j / S1N) & 1, abort_flag, p.err, ERR_WAIT_FULL)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t da = make_smem_desc(r1_s + (kk >> 2) * R_SUB + (kk & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(s1_s + st1 * S_BYTES + (kk >> 2) * S_SUB + (kk & 3) * 32, 16, 1024);
          umma_f16(tmem_base + buf * BN, da, db, idesc_fs, kk != 0);
        }
        if (!TWO) umma_commit(bar(B_S1E + st1));
        umma_commit(bar(B_SPF + buf));
        return true;
      };
      if (ok) ok = first_stage(0);
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          ok = first_stage(j + 1);
          if (!ok) break;
        }
        const int buf = j & 1, st1 = j % S1N, st2 = j % S2N;
        if (!TWO) {
          ok = mbar_wait(bar(B_S2F + st2), (j / S2N) & 1, abort_flag, p.err, ERR_WAIT_FULL);
          if (!ok) break;
        }
        ok = mbar_wait(bar(B_TRD + buf), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_FULL);
        if (!ok) break;
        tc_fence_after();
        const uint32_t b_tile = TWO ? s1_s + st1 * S_BYTES : s2_s + st2 * S_BYTES;
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          const uint64_t db = make_smem_desc(b_tile + ks * 2048, S_SUB, 1024);
          umma_f16_ts(tmem_base + ACC_COL, tmem_base + buf * BN + ks * 8, db, idesc_ss, (j | ks) != 0);
        }
        umma_commit(bar(TWO ? B_S1E + st1 : B_S2E + st2));
      }
      if (ok) umma_commit(bar(B_ACC));
    }
  } else {
    // ------------------------------------------------------------------ transform (thread = resident row) + epilogue
    const int quad = warp & 3;
    const int row_l = quad * 32 + lane;
    const int row = row0 + row_l;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const float sc = p.scale * FA_LOG2E;
    const bool fp16 = p.fp16 != 0;
    const uint8_t* kpm_b = p.kpm ? p.kpm + static_cast<long long>(b) * p.Sk : nullptr;
    // statistics of a query row (dQ); whether this key row is padding (dK, dV)
    float lse2_r = CUDART_INF_F, delta_r = 0.f;
    bool row_keep = true;
    if (KEY_ROWS) {
      row_keep = row < p.Sk && (!kpm_b || kpm_b[row] != 0);
    } else if (row < p.Sq) {
      lse2_r = p.lse[stat_base + row] * FA_LOG2E;
      delta_r = p.delta[stat_base + row];
    }
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      const int buf = j & 1;
      const int c0 = c_lo + j * BN;
      ok = mbar_wait(bar(B_SPF + buf), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      if (KEY_ROWS) {
        ok = mbar_wait(bar(B_STF + buf), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_FULL);
        if (!ok) break;
      }
      tc_fence_after();
      float s[BN];
#pragma unroll
      for (int cc = 0; cc < BN; cc += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_lane + buf * BN + cc, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[cc + i] = __uint_as_float(r[i]) * sc;
      }
      const float* sb = stats + buf * 2 * BN;
      // ---- P (or P^T)
#pragma unroll
      for (int i = 0; i < BN; ++i) {
        const float l2 = KEY_ROWS ? sb[i] : lse2_r;
        s[i] = exp2f(s[i] - l2);
      }
      bool need_mask;
      if (KEY_ROWS)
        need_mask = (p.causal && row0 + FA_BM - 1 > c0 + offset) || (p.window > 0 && row0 <= c0 + BN - 1 + offset - p.window);
      else
        need_mask = (c0 + BN > p.Sk) || kpm_b != nullptr || (p.causal && c0 + BN - 1 > row0 + offset) ||
                    (p.window > 0 && c0 <= row0 + FA_BM - 1 + offset - p.window);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int q = KEY_ROWS ? c0 + i : row;
          const int k = KEY_ROWS ? row : c0 + i;
          bool vis = fa_visible(q, k, offset, p.Sq, p.Sk, p.causal, p.window);
          if (!KEY_ROWS && vis && kpm_b && !kpm_b[k]) vis = false;
          if (!vis) s[i] = 0.f;
        }
      }
      if (KEY_ROWS && !row_keep) {
#pragma unroll
        for (int i = 0; i < BN; ++i) s[i] = 0.f;
      }
      if (TWO) {
        // ---- dS = P o (dP - delta)
#pragma unroll
        for (int cc = 0; cc < BN; cc += 32) {
          uint32_t r[32];
          tmem_ld_32x32(t_lane + DP_COL + buf * BN + cc, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float dl = KEY_ROWS ? sb[BN + cc + i] : delta_r;
            s[cc + i] *= (__uint_as_float(r[i]) - dl);
          }
        }
      }
      // ---- 16-bit tile back into the S columns it came from (two elements per 32-bit column)
#pragma unroll
      for (int cc = 0; cc < BN / 2; cc += 32) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = fa_pack2(s[2 * (cc + i)], s[2 * (cc + i) + 1], fp16);
        tmem_st_32x32(t_lane + buf * BN + cc, r);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_TRD + buf));
    }
    // ---- epilogue: accumulator (x scale for dK, dQ) -> global
    if (ok && nblk > 0) {
      ok = mbar_wait(bar(B_ACC), 0, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      tc_fence_after();
    }
    const float mult = TWO ? p.scale : 1.f;
    uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + b * p.o_sb + h * p.o_sh + static_cast<long long>(row) * p.o_ss;
#pragma unroll 1
    for (int cc = 0; cc < D; cc += 32) {
      uint32_t r[32];
      if (nblk > 0 && ok) {
        tmem_ld_32x32(t_lane + ACC_COL + cc, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      if (row < n_rows) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          v.x = fa_pack2(__uint_as_float(r[i]) * mult, __uint_as_float(r[i + 1]) * mult, fp16);
          v.y = fa_pack2(__uint_as_float(r[i + 2]) * mult, __uint_as_float(r[i + 3]) * mult, fp16);
          v.z = fa_pack2(__uint_as_float(r[i + 4]) * mult, __uint_as_float(r[i + 5]) * mult, fp16);
          v.w = fa_pack2(__uint_as_float(r[i + 6]) * mult, __uint_as_float(r[i + 7]) * mult, fp16);
          *reinterpret_cast<uint4*>(orow + cc + i) = v;
        }
      }
    }
  }

  if (*abort_flag) {  // let copies that are still in flight land before the shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------- host side
template <int D, int BN, int MODE, int S1N, int S2N>
static int fa_bwd_launch(const CUtensorMap& tr1, const CUtensorMap& tr2, const CUtensorMap& ts1, const CUtensorMap& ts2,
                         const FaBwdParams& p, cudaStream_t stream) {
  constexpr int NRES = MODE != BWD_DV ? 2 : 1;
  constexpr int NBAR = 1 + 2 * S1N + 2 * S2N + 7;
  constexpr size_t smem = NRES * FA_BM * D * 2 + (S1N + S2N) * BN * D * 2 + (MODE != BWD_DQ ? 16 * BN : 0) + NBAR * 8 + 16 + 1024;
  static_assert(smem <= 232448, "shared memory budget of one CTA");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(fa_bwd_kernel<D, BN, MODE, S1N, S2N>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int rows = MODE != BWD_DQ ? p.Sk : p.Sq;
  dim3 grid((rows + FA_BM - 1) / FA_BM, p.H, p.B);
  fa_bwd_kernel<D, BN, MODE, S1N, S2N><<<grid, FA_THREADS, smem, stream>>>(tr1, tr2, ts1, ts2, p);
  return static_cast<int>(cudaGetLastError());
}

template <int D, int BN_DV, int S1N, int S2N>
static int fa_bwd_all(const void* q, const void* k, const void* v, const void* dout, void* dq, void* dk, void* dv,
                      FaBwdParams p, int B, int H, int Sq, int Sk, const long long* qs, const long long* ks,
                      const long long* vs, const long long* ds, bool fp16, cudaStream_t stream) {
  CUtensorMap tr1, tr2, ts1, ts2;
  int rc;
  // ---- dV: resident K, streamed Q (first stage) and dO (second stage)
  if ((rc = make_qkv_map(&tr1, k, B, H, Sk, D, ks[0], ks[1], ks[2], FA_BM, fp16, p.r1_pos))) return rc;
  if ((rc = make_qkv_map(&ts1, q, B, H, Sq, D, qs[0], qs[1], qs[2], BN_DV, fp16, p.s1_pos))) return rc;
  if ((rc = make_qkv_map(&ts2, dout, B, H, Sq, D, ds[0], ds[1], ds[2], BN_DV, fp16, p.s2_pos))) return rc;
  p.out = dv; p.o_sb = vs[0]; p.o_sh = vs[1]; p.o_ss = vs[2];
  if ((rc = fa_bwd_launch<D, BN_DV, BWD_DV, 2, 2>(tr1, tr1, ts1, ts2, p, stream))) return rc;
  // ---- dK: resident K and V, streamed Q (both stages) and dO
  if ((rc = make_qkv_map(&tr2, v, B, H, Sk, D, vs[0], vs[1], vs[2], FA_BM, fp16, p.r2_pos))) return rc;
  if ((rc = make_qkv_map(&ts1, q, B, H, Sq, D, qs[0], qs[1], qs[2], 64, fp16, p.s1_pos))) return rc;
  if ((rc = make_qkv_map(&ts2, dout, B, H, Sq, D, ds[0], ds[1], ds[2], 64, fp16, p.s2_pos))) return rc;
  p.out = dk; p.o_sb = ks[0]; p.o_sh = ks[1]; p.o_ss = ks[2];
  if ((rc = fa_bwd_launch<D, 64, BWD_DK, S1N, S2N>(tr1, tr2, ts1, ts2, p, stream))) return rc;
  // ---- dQ: resident Q and dO, streamed K (both stages) and V
  if ((rc = make_qkv_map(&tr1, q, B, H, Sq, D, qs[0], qs[1], qs[2], FA_BM, fp16, p.r1_pos))) return rc;
  if ((rc = make_qkv_map(&tr2, dout, B, H, Sq, D, ds[0], ds[1], ds[2], FA_BM, fp16, p.r2_pos))) return rc;
  if ((rc = make_qkv_map(&ts1, k, B, H, Sk, D, ks[0], ks[1], ks[2], 64, fp16, p.s1_pos))) return rc;
  if ((rc = make_qkv_map(&ts2, v, B, H, Sk, D, vs[0], vs[1], vs[2], 64, fp16, p.s2_pos))) return rc;
  p.out = dq; p.o_sb = qs[0]; p.o_sh = qs[1]; p.o_ss = qs[2];
  return fa_bwd_launch<D, 64, BWD_DQ, S1N, S2N>(tr1, tr2, ts1, ts2, p, stream);
}

}  // namespace oslo

// dq / dk / dv use the strides of q / k / v. `delta` is a [B, H, Sq] fp32 workspace. Four launches.
extern "C" int oslo_flash_bwd_sm100(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                    const float* lse, float* delta, void* dq, void* dk, void* dv, const uint8_t* kpm,
                                    int B, int H, int Sq, int Sk, int D, long long q_sb, long long q_sh, long long q_ss,
                                    long long k_sb, long long k_sh, long long k_ss, long long v_sb, long long v_sh,
                                    long long v_ss, long long o_sb, long long o_sh, long long o_ss, long long do_sb,
                                    long long do_sh, long long do_ss, float scale, int causal, int window, int dtype,
                                    int* err_word, cudaStream_t stream) {
  using namespace oslo;
  if (B <= 0 || H <= 0 || Sq <= 0 || Sk <= 0) return -1;
  if (D != 64 && D != 128 && D != 256) return -2;
  if (dtype != OSLO_DT_BF16 && dtype != OSLO_DT_FP16) return -3;
  const void* outs[3] = {dq, dk, dv};
  for (const void* ptr : outs)
    if (reinterpret_cast<uintptr_t>(ptr) & 15) return -4;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(nullptr); ctx_bound = true; }
  const bool fp16 = dtype == OSLO_DT_FP16;
  {
    const long long rows = static_cast<long long>(B) * H * Sq;
    const int wpb = 8;
    const unsigned blocks = static_cast<unsigned>((rows + wpb - 1) / wpb);
    if (fp16)
      fa_delta_kernel<__half><<<blocks, wpb * 32, 0, stream>>>(static_cast<const __half*>(o), static_cast<const __half*>(dout),
                                                               delta, B, H, Sq, D, o_sb, o_sh, o_ss, do_sb, do_sh, do_ss);
    else
      fa_delta_kernel<__nv_bfloat16><<<blocks, wpb * 32, 0, stream>>>(static_cast<const __nv_bfloat16*>(o),
                                                                      static_cast<const __nv_bfloat16*>(dout), delta, B, H,
                                                                      Sq, D, o_sb, o_sh, o_ss, do_sb, do_sh, do_ss);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  FaBwdParams p{};
  p.lse = lse; p.delta = delta; p.kpm = kpm;
  p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk;
  p.scale = scale; p.causal = causal; p.window = window; p.fp16 = fp16 ? 1 : 0; p.err = err_word;
  const long long qs[3] = {q_sb, q_sh, q_ss}, ks[3] = {k_sb, k_sh, k_ss}, vs[3] = {v_sb, v_sh, v_ss},
                  ds[3] = {do_sb, do_sh, do_ss};
  if (D == 64) return fa_bwd_all<64, 128, 3, 2>(q, k, v, dout, dq, dk, dv, p, B, H, Sq, Sk, qs, ks, vs, ds, fp16, stream);
  if (D == 128) return fa_bwd_all<128, 128, 3, 2>(q, k, v, dout, dq, dk, dv, p, B, H, Sq, Sk, qs, ks, vs, ds, fp16, stream);
  return fa_bwd_all<256, 64, 2, 1>(q, k, v, dout, dq, dk, dv, p, B, H, Sq, Sk, qs, ks, vs, ds, fp16, stream);
}
