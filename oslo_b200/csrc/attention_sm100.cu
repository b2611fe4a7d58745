// Flash attention on the 5th-generation tensor cores (tcgen05 + TMEM), forward pass.
//
// One CTA owns 128 query rows of one (batch, head); one TMEM lane per row. 192 threads:
//   warp 0     TMA producer: Q once, then K and V blocks through two 2-deep shared-memory rings
//   warp 1     TMEM owner + the single MMA-issuing lane
//   warps 2-5  softmax: thread = query row. They read S = Q K^T from TMEM (tcgen05.ld), apply the mask
//              (causal with query offset, sliding window, key padding), keep the running max / sum, write
//              P = exp2(S - m) as 16-bit pairs back into the TMEM columns S came from (the next MMA reads its A
//              operand from tensor memory; a shared-memory P tile in the 128-byte-swizzled K-major layout is
//              the alternative path), and rescale the O accumulator in TMEM only when the running max has grown
//              by more than 2^8 (warp-uniform decision), so most blocks never touch O.
// S is double-buffered in TMEM so Q K^T of block j+1 runs under the softmax of block j, and P V of block j runs
// under the softmax of block j+1. O (128 x D fp32) stays in TMEM for the whole row of blocks.
// The K tile [BN x 64]-column sub-tiles are at the same time the MN-major image of V that P V needs, so K and V
// use the same TMA box and no transposes exist anywhere. Every wait is bounded (ptx.cuh).
//
// Reference behaviour covered: the materialised-score path Q K^T -> scaled (upper-triangular | padding) masked
// softmax -> P V of oslo/models/gptj/modeling_gptj.py:151-191 with the kernels of
// oslo/fused_kernels/includes/fused_triang_softmax.h:134-351 and fused_softmax.h:111-325 (sequence length <= 2048
// there; no limit here), plus GPT-Neo's local window (oslo/models/gpt_neo/modeling_gpt_neo.py:150-160).
#include "attention_sm100.cuh"

namespace oslo {

constexpr float FA_RESCALE_THRESHOLD = 8.0f;  // log2 units

struct FaParams {
  void* out;          // [B, H, Sq, D] element strides below
  float* lse;         // [B, H, Sq]
  const uint8_t* kpm; // [B, Sk] 1 = keep, or nullptr
  int B, H, Sq, Sk;
  long long o_sb, o_sh, o_ss;
  float scale;
  int causal, window;
  int fp16;
  // position of the (seq, head, batch) coordinates inside each 4-D tensor map (dim 0 is always D)
  int q_pos[3], k_pos[3], v_pos[3];
  int* err;
};

// PT = true: P goes back into TMEM (over the S buffer it came from, two bf16 per 32-bit column) and is the
// A operand of P V straight from tensor memory; PT = false: P goes through a swizzled shared-memory tile.
template <int D, int BN, bool PT>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
              const __grid_constant__ CUtensorMap tv, const FaParams p) {
  constexpr int DC = D / 64;                     // 64-column sub-tiles per row operand
  constexpr uint32_t Q_SUB = FA_BM * 128;        // bytes of one [128 x 64] sub-tile (Q and P)
  constexpr uint32_t KV_SUB = BN * 128;          // bytes of one [BN x 64] sub-tile (K and V)
  constexpr uint32_t Q_BYTES = DC * Q_SUB;
  constexpr uint32_t KV_BYTES = DC * KV_SUB;
  constexpr uint32_t P_BYTES = PT ? 0u : (BN / 64) * Q_SUB;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t O_COL = 2 * BN;             // S buffers at columns [0, BN) and [BN, 2 BN)
  static_assert(O_COL + D <= TMEM_COLS, "TMEM budget");

  extern __shared__ uint8_t fa_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fa_smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t q_s = smem_u32(smem);
  const uint32_t k_s = q_s + Q_BYTES;            // 2 stages
  const uint32_t v_s = k_s + 2 * KV_BYTES;       // 2 stages
  const uint32_t p_s = v_s + 2 * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Q_BYTES + 4 * KV_BYTES + P_BYTES);
  const uint32_t bar0 = smem_u32(bars);
  // 0 q_full | 1,2 k_full | 3,4 k_empty | 5,6 v_full | 7,8 v_empty | 9,10 s_full | 11,12 s_empty | 13 p_ready[0] |
  // 14 pv_done | 15 p_ready[1] (PT only: one per S/P buffer)
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y;
  const int q0 = (static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x)) * FA_BM;  // long (late) rows first
  const int offset = p.Sk - p.Sq;
  int key_hi = p.Sk, key_lo = 0;
  if (p.causal) key_hi = min(p.Sk, q0 + FA_BM + offset);
  if (p.window > 0) key_lo = max(0, q0 + offset - p.window + 1) / BN * BN;
  const int nblk = key_hi > key_lo ? (key_hi - key_lo + BN - 1) / BN : 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 16; ++i) {
      const bool four = (i == 11 || i == 12 || i == 13 || i == 15);  // arrivals from the 4 softmax warps
      mbar_init(bar(i), four ? 4 : 1);
    }
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && nblk > 0) {
      tma_prefetch_desc(&tq); tma_prefetch_desc(&tk); tma_prefetch_desc(&tv);
      mbar_expect_tx(bar(0), Q_BYTES);
#pragma unroll
      for (int c = 0; c < DC; ++c) tma_load_rows(q_s + c * Q_SUB, &tq, bar(0), c * 64, q0, h, b, p.q_pos);
      bool ok = true;
      for (int j = 0; j < nblk && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int n0 = key_lo + j * BN;
        ok = mbar_wait(bar(3 + st), ph ^ 1, abort_flag, p.err, ERR_WAIT_EMPTY);
        if (!ok) break;
        mbar_expect_tx(bar(1 + st), KV_BYTES);
#pragma unroll
        for (int c = 0; c < DC; ++c) tma_load_rows(k_s + st * KV_BYTES + c * KV_SUB, &tk, bar(1 + st), c * 64, n0, h, b, p.k_pos);
        ok = mbar_wait(bar(7 + st), ph ^ 1, abort_flag, p.err, ERR_WAIT_EMPTY);
        if (!ok) break;
        mbar_expect_tx(bar(5 + st), KV_BYTES);
#pragma unroll
        for (int c = 0; c < DC; ++c) tma_load_rows(v_s + st * KV_BYTES + c * KV_SUB, &tv, bar(5 + st), c * 64, n0, h, b, p.v_pos);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && nblk > 0) {
      const int fmt = p.fp16 ? 0 : 1;
      const uint32_t idesc_qk = make_idesc_f16(FA_BM, BN, fmt, 0, 0);
      const uint32_t idesc_pv = make_idesc_f16(FA_BM, D, fmt, 0, 1);
      bool ok = mbar_wait(bar(0), 0, abort_flag, p.err, ERR_WAIT_FULL);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(bar(1 + st), ph, abort_flag, p.err, ERR_WAIT_FULL)) return false;
        if (!mbar_wait(bar(11 + st), ph ^ 1, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t da = make_smem_desc(q_s + (kk >> 2) * Q_SUB + (kk & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(k_s + st * KV_BYTES + (kk >> 2) * KV_SUB + (kk & 3) * 32, 16, 1024);
          umma_f16(tmem_base + st * BN, da, db, idesc_qk, kk != 0);
        }
        umma_commit(bar(3 + st));   // K stage may be refilled once these MMAs have read it
        umma_commit(bar(9 + st));   // S_j is ready for the softmax warps
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < nblk && ok; ++j) {
        if (j + 1 < nblk) {
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        const int st = j & 1;
        ok = mbar_wait(bar(5 + st), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_FULL);
        if (!ok) break;
        if (PT) ok = mbar_wait(bar(st ? 15 : 13), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_FULL);
        else ok = mbar_wait(bar(13), j & 1, abort_flag, p.err, ERR_WAIT_FULL);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          const uint64_t db = make_smem_desc(v_s + st * KV_BYTES + ks * 2048, KV_SUB, 1024);
          if (PT) {
            umma_f16_ts(tmem_base + O_COL, tmem_base + st * BN + ks * 8, db, idesc_pv, (j | ks) != 0);
          } else {
            const uint64_t da = make_smem_desc(p_s + (ks >> 2) * Q_SUB + (ks & 3) * 32, 16, 1024);
            umma_f16(tmem_base + O_COL, da, db, idesc_pv, (j | ks) != 0);
          }
        }
        umma_commit(bar(7 + st));   // V stage free
        umma_commit(bar(14));       // O updated, P buffer reusable
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const int quad = warp & 3;
    const int row_l = quad * 32 + lane;
    const int row = q0 + row_l;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint8_t* kpm_row = p.kpm ? p.kpm + static_cast<long long>(b) * p.Sk : nullptr;
    const float sc = p.scale * FA_LOG2E;
    const bool fp16 = p.fp16 != 0;
    float m_ref = -CUDART_INF_F, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      const int st = j & 1;
      const int n0 = key_lo + j * BN;
      ok = mbar_wait(bar(9 + st), (j >> 1) & 1, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      tc_fence_after();
      float s[BN];
#pragma unroll
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(t_lane + st * BN + c0, r);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[c0 + i] = __uint_as_float(r[i]) * sc;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(11 + st));  // S buffer may be overwritten by Q K^T of block j + 2
      // ---- mask (only blocks that touch the diagonal, the window edge, the end of the keys, or padding)
      const bool need_mask = (n0 + BN > p.Sk) || kpm_row != nullptr ||
                             (p.causal && n0 + BN - 1 > q0 + offset) ||
                             (p.window > 0 && n0 <= q0 + FA_BM - 1 + offset - p.window);
      if (need_mask) {
        const int qpos = row + offset;
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int col = n0 + i;
          bool vis = col < p.Sk;
          if (p.causal && col > qpos) vis = false;
          if (p.window > 0 && col <= qpos - p.window) vis = false;
          if (vis && kpm_row && !kpm_row[col]) vis = false;
          if (!vis) s[i] = -CUDART_INF_F;
        }
      }
      // four independent chains: one thread per row means nothing else hides the latency of a 64-long dependent chain
      float mx4[4] = {s[0], s[1], s[2], s[3]};
#pragma unroll
      for (int i = 4; i < BN; i += 4) {
        mx4[0] = fmaxf(mx4[0], s[i]);
        mx4[1] = fmaxf(mx4[1], s[i + 1]);
        mx4[2] = fmaxf(mx4[2], s[i + 2]);
        mx4[3] = fmaxf(mx4[3], s[i + 3]);
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_ref, mx);
      // rescale O only when some row of this warp outgrew its reference by 2^8 (or on the first block)
      const bool grow = (j == 0) || (m_new - m_ref > FA_RESCALE_THRESHOLD);
      const bool rescale = __any_sync(0xffffffffu, grow);
      float factor = 1.f;
      if (rescale) {
        factor = (m_ref == -CUDART_INF_F) ? 0.f : exp2f(m_ref - m_new);
        m_ref = m_new;
        l_sum *= factor;
      }
      const float m_use = (m_ref == -CUDART_INF_F) ? 0.f : m_ref;
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < BN; i += 4) {
        s[i] = exp2f(s[i] - m_use);
        s[i + 1] = exp2f(s[i + 1] - m_use);
        s[i + 2] = exp2f(s[i + 2] - m_use);
        s[i + 3] = exp2f(s[i + 3] - m_use);
        ps4[0] += s[i];
        ps4[1] += s[i + 1];
        ps4[2] += s[i + 2];
        ps4[3] += s[i + 3];
      }
      l_sum += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      // the shared P tile is single-buffered, so P V of block j-1 must have finished before it is rewritten; the
      // TMEM P buffers alternate, so there only a rescale of O has to wait for it
      if (j > 0 && (!PT || rescale)) {
        ok = mbar_wait(bar(14), (j - 1) & 1, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
        if (!ok) break;
        tc_fence_after();
        if (rescale) {
#pragma unroll 1
          for (int c0 = 0; c0 < D; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32(t_lane + O_COL + c0, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * factor);
            tmem_st_32x32(t_lane + O_COL + c0, r);
          }
          tmem_wait_st();
        }
      }
      if constexpr (PT) {
#pragma unroll
        for (int c0 = 0; c0 < BN / 2; c0 += 32) {
          uint32_t r[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = fa_pack2(s[2 * (c0 + i)], s[2 * (c0 + i) + 1], fp16);
          tmem_st_32x32(t_lane + st * BN + c0, r);
        }
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(st ? 15 : 13));
      } else {
      // ---- P (bf16) into shared memory: K-major, 128-byte swizzle: 16-byte chunk c of row r sits at c ^ (r & 7)
#pragma unroll
      for (int c = 0; c < BN / 64; ++c) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int i0 = c * 64 + q * 8;
          uint4 v;
          v.x = fa_pack2(s[i0], s[i0 + 1], fp16); v.y = fa_pack2(s[i0 + 2], s[i0 + 3], fp16);
          v.z = fa_pack2(s[i0 + 4], s[i0 + 5], fp16); v.w = fa_pack2(s[i0 + 6], s[i0 + 7], fp16);
          const uint32_t addr = p_s + c * Q_SUB + row_l * 128 + ((q ^ (row_l & 7)) << 4);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
        }
      }
      fence_proxy_async_smem();   // generic-proxy writes -> visible to the tensor core's async proxy
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(13));
      }
    }
    // ---- epilogue: O / l -> global, log-sum-exp
    if (ok && nblk > 0) {
      ok = mbar_wait(bar(14), (nblk - 1) & 1, abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      tc_fence_after();
    }
    const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
    uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + b * p.o_sb + h * p.o_sh + static_cast<long long>(row) * p.o_ss;
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t r[32];
      if (nblk > 0 && ok) {
        tmem_ld_32x32(t_lane + O_COL + c0, r);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = 0u;
      }
      if (row < p.Sq) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 v;
          v.x = fa_pack2(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv, fp16);
          v.y = fa_pack2(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv, fp16);
          v.z = fa_pack2(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv, fp16);
          v.w = fa_pack2(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv, fp16);
          *reinterpret_cast<uint4*>(orow + c0 + i) = v;
        }
      }
    }
    if (row < p.Sq && p.lse) {
      const float lse = l_sum > 0.f ? (m_ref + log2f(l_sum)) * FA_LN2 : 0.f;
      p.lse[(static_cast<long long>(b) * p.H + h) * p.Sq + row] = lse;
    }
  }

  if (*abort_flag) {
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
template <int D, int BN, bool PT>
static int fa_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p,
                     cudaStream_t stream) {
  constexpr size_t smem = FA_BM * D * 2 + 4 * BN * D * 2 + (PT ? 0 : FA_BM * BN * 2) + 16 * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(fa_fwd_kernel<D, BN, PT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  dim3 grid((p.Sq + FA_BM - 1) / FA_BM, p.H, p.B);
  fa_fwd_kernel<D, BN, PT><<<grid, FA_THREADS, smem, stream>>>(tq, tk, tv, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace oslo

extern "C" int oslo_flash_fwd_sm100(const void* q, const void* k, const void* v, void* o, float* lse,
                                    const uint8_t* kpm, int B, int H, int Sq, int Sk, int D, long long q_sb,
                                    long long q_sh, long long q_ss, long long k_sb, long long k_sh, long long k_ss,
                                    long long v_sb, long long v_sh, long long v_ss, long long o_sb, long long o_sh,
                                    long long o_ss, float scale, int causal, int window, int dtype, int* err_word,
                                    cudaStream_t stream) {
  using namespace oslo;
  if (B <= 0 || H <= 0 || Sq <= 0 || Sk <= 0) return -1;
  if (D != 64 && D != 128 && D != 256) return -2;
  if (dtype != OSLO_DT_BF16 && dtype != OSLO_DT_FP16) return -3;
  if ((reinterpret_cast<uintptr_t>(o) & 15) || (o_sb % 8) || (o_sh % 8) || (o_ss % 8)) return -4;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(nullptr); ctx_bound = true; }
  const bool fp16 = dtype == OSLO_DT_FP16;
  const int bn = D == 256 ? 64 : 128;
  FaParams p;
  p.out = o; p.lse = lse; p.kpm = kpm;
  p.B = B; p.H = H; p.Sq = Sq; p.Sk = Sk;
  p.o_sb = o_sb; p.o_sh = o_sh; p.o_ss = o_ss;
  p.scale = scale; p.causal = causal; p.window = window; p.fp16 = fp16 ? 1 : 0; p.err = err_word;
  CUtensorMap tq, tk, tv;
  int rc = make_qkv_map(&tq, q, B, H, Sq, D, q_sb, q_sh, q_ss, FA_BM, fp16, p.q_pos);
  if (rc) return rc;
  rc = make_qkv_map(&tk, k, B, H, Sk, D, k_sb, k_sh, k_ss, bn, fp16, p.k_pos);
  if (rc) return rc - 1000;
  rc = make_qkv_map(&tv, v, B, H, Sk, D, v_sb, v_sh, v_ss, bn, fp16, p.v_pos);
  if (rc) return rc - 2000;
  static const bool p_smem = [] { const char* e = getenv("OSLO_B200_ATTN_P_SMEM"); return e && e[0] == '1'; }();
  if (p_smem) {
    if (D == 64) return fa_launch<64, 128, false>(tq, tk, tv, p, stream);
    if (D == 128) return fa_launch<128, 128, false>(tq, tk, tv, p, stream);
    return fa_launch<256, 64, false>(tq, tk, tv, p, stream);
  }
  if (D == 64) return fa_launch<64, 128, true>(tq, tk, tv, p, stream);
  if (D == 128) return fa_launch<128, 128, true>(tq, tk, tv, p, stream);
  return fa_launch<256, 64, true>(tq, tk, tv, p, stream);
}
