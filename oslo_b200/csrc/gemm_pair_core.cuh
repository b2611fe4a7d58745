// tcgen05 GEMM on CTA pairs (cluster of two SMs, cta_group::2): one 256 x 256 output tile per pair.
//
// Each CTA stages 128 rows of A and 128 of the tile's 256 B rows per k-block (32 KB instead of the 48 KB a
// 128 x 256 single-CTA tile needs), so the same shared memory holds a deeper ring and every SM pulls a third
// less operand data out of L2 per FLOP. The even CTA of the pair issues the MMAs (M = 256: each CTA's tensor
// core multiplies its own A rows by the B rows of BOTH CTAs and accumulates into its own TMEM); both CTAs run a
// TMA producer and four epilogue warps. Barrier traffic between the two CTAs:
//   full[s]    lives in the even CTA; both producers' TMA copies count their bytes on it
//   empty[s]   one per CTA; the MMA thread commits to both
//   tfull[b]   one per CTA; the MMA thread commits to both
//   tempty[b]  lives in the even CTA; 8 arrivals (4 epilogue warps of each CTA)
// Each CTA fetches exactly the boxes it consumes itself. Every wait is bounded (ptx.cuh); the two
// cluster-wide barriers (after set-up, before tear-down) are reached unconditionally by every thread.
//
// Reference behaviour covered: every torch.matmul of the parallel layers (oslo/modeling_utils.py:63-104) and their
// autograd gradients; the reference has no GEMM kernel of its own.
#pragma once
#include "gemm_core.cuh"

namespace oslo {

constexpr int PAIR_TILE = 256;  // output tile edge of a pair (M and N)

template <int STAGES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                         const GemmParams p) {
  constexpr uint32_t A_BYTES = BM * BK * 2;       // this CTA's 128 rows of A
  constexpr uint32_t B_BYTES = BM * BK * 2;       // this CTA's 128 of the 256 B rows
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * PAIR_TILE;   // two accumulators of 256 columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0 = even CTA (issues the MMAs), 1 = its peer
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();   // the peer's barriers exist before anything of this CTA can signal them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;    // 256 x 256 tiles
  const int kblocks = (p.K + BK - 1) / BK;
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += n_clusters) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn, p.group_m);
        const int m0 = tm * PAIR_TILE + static_cast<int>(rank) * BM;
        const int n0 = tn * PAIR_TILE + static_cast<int>(rank) * BM;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, p.err, ERR_WAIT_EMPTY);
          if (!ok) break;
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const uint32_t fb = map_to_cta(full_bar(stage), 0);
          if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);   // both CTAs' bytes
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_2d_pair(sa, &tma_a, fb, k0, m0);                        // box {64 k, 128 rows}
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)                                // boxes {64 m, 64 k rows}
              tma_load_2d_pair(sa + c * 8192, &tma_a, fb, m0 + c * 64, k0);
          }
          if (!p.b_mn_major) {
            tma_load_2d_pair(sb, &tma_b, fb, k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d_pair(sb + c * 8192, &tma_b, fb, n0 + c * 64, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (even CTA only)
    if (lane == 0 && rank == 0) {
      const int fmt = (p.flags & GEMM_FLAG_FP16) ? 0 : 1;
      const uint32_t idesc = make_idesc_f16(PAIR_TILE, PAIR_TILE, fmt, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, a_step = p.a_mn_major ? 2048u : 32u;
      const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u, b_step = p.b_mn_major ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += n_clusters, ++local) {
        const int buf = local & 1;
        ok = mbar_wait(tempty_bar(buf), acc_phase[buf] ^ 1, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        acc_phase[buf] ^= 1;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * PAIR_TILE;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(full_bar(stage), phase, abort_flag, p.err, ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = make_smem_desc(sa + k * a_step, a_lbo, 1024);
            const uint64_t db = make_smem_desc(sb + k * b_step, b_lbo, 1024);
            umma_f16_pair(tmem_acc, da, db, idesc, (kb | k) != 0);
          }
          umma_commit_pair(empty_bar(stage));                  // this CTA's stage ...
          umma_commit_pair(map_to_cta(empty_bar(stage), 1));   // ... and the peer's
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) {
          umma_commit_pair(tfull_bar(buf));
          umma_commit_pair(map_to_cta(tfull_bar(buf), 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quad = warp & 3;
    const bool fp16 = (p.flags & GEMM_FLAG_FP16) != 0;
    const bool out_f32 = (p.flags & GEMM_FLAG_OUT_FP32) != 0;
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += n_clusters, ++local) {
      const int buf = local & 1;
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn, p.group_m);
      ok = mbar_wait(tfull_bar(buf), acc_phase[buf], abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      acc_phase[buf] ^= 1;
      tc_fence_after();
      const int row = tm * PAIR_TILE + static_cast<int>(rank) * BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * PAIR_TILE;
      const bool ce_stats = (p.flags & GEMM_FLAG_CE_STATS) != 0;
      CeAcc ce;
      ce_reset(ce);
      const long long label_local = (ce_stats && row_ok) ? p.ce_labels[row] - p.ce_vocab_start : -1;
#pragma unroll 1
      for (int c0 = 0; c0 < PAIR_TILE; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_wait_ld();
        const int col0 = tn * PAIR_TILE + c0;
        if (!row_ok || col0 >= p.N) continue;
        if (ce_stats) {
          ce_accumulate(p, col0, r, fp16, label_local, ce);
          ce_flush_if_block_ends(p, row, col0, ce);
        } else {
          epilogue_chunk(p, row, col0, r, fp16, out_f32);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0));
    }
  }

  if (*abort_flag) {  // let copies that are still in flight land before the shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) {
    }
  }
  tc_fence_before();
  cluster_sync_all();   // nothing of the peer may still be signalling this CTA's barriers or reading its tiles
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace oslo
