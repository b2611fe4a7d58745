// GEMM fused with a tensor-parallel collective over NVLink / NVSwitch, ONE kernel per op:
//
//   COMM_ALLREDUCE       D = sum over ranks of (A_r x B_r^T)            row-parallel forward, column-parallel dgrad
//   COMM_REDUCE_SCATTER  D_r = rows r of that sum                        sequence-parallel row-parallel forward
//   COMM_ALLGATHER_A     D = [A_0; A_1; ...] x B^T with A_r on rank r    sequence-parallel column-parallel forward
//
// The tcgen05 main loop is the one of gemm_core.cuh; four extra warps per CTA do the traffic while the
// tensor cores work on other tiles:
//   * reduce modes: the epilogue stores this rank's partial tile into its symmetric buffer and bumps a flag
//     on the rank that owns the tile; the owner's communication warps wait (bounded) for `world` arrivals,
//     pull the sum with multimem.ld_reduce (the switch adds the ranks' copies) - or with plain peer loads when
//     no multicast mapping exists - and either store it locally (reduce-scatter) or broadcast it back with
//     multimem.st (all-reduce), then count the tile as final on every rank;
//   * all-gather mode: communication warps copy this rank's shard into every rank's gather buffer chunk by
//     chunk and raise per-chunk flags; the TMA warp waits for the chunk a tile needs before loading it - from
//     LOCAL memory, with a plain (non-multicast) TMA load. Row blocks are walked starting at the local shard.
// Flags are epoch-counted and never reset; the caller cycles through several workspace slots so a fast rank cannot
// overwrite data a slow rank still reads: a rank can finish call c + k only when every peer has at least started
// call c + k, so it reaches the call that reuses a slot after every peer has issued all but the last of the calls
// in between. A wait that runs out records ERR_WAIT_PEER and the kernel tears down normally.
#include <cstdlib>

#include "gemm_core.cuh"

namespace oslo {
int make_tma_2d_16bit(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_rows, bool fp16);

template <int BN, int STAGES>
static int launch_comm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int num_sms, cudaStream_t stream) {
  constexpr size_t smem = STAGES * (BM * BK * 2 + BN * BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  // every rank must launch the same grid: tile ownership and the work split of the communication warps depend on it
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_tcgen05_kernel<BN, STAGES, true><<<grid, GEMM_THREADS_COMM, smem, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}
}  // namespace oslo

extern "C" int oslo_gemm_comm_16bit(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int a_mn_major,
                                    int b_mn_major, const void* bias, const void* aux, int ld_aux, void* aux_out, int ld_aux_out, int flags,
                                    float alpha, void* const* peer_bufs_dev, void* own_buf, void* mc_base,
                                    long long data_off, long long flag_off, long long flag_bytes, int rank, int world,
                                    unsigned epoch, unsigned done_base, int mode, int use_multimem, void* out,
                                    int ld_out, int wide_tiles, unsigned long long* trace, int* err_word, int num_sms,
                                    cudaStream_t stream) {
  using namespace oslo;
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || rank < 0 || rank >= world) return -1;
  if (N % 8 || K % 8) return -3;
  if (mode != COMM_ALLREDUCE && (M % (world * BM))) return -5;  // row ownership must fall on tile boundaries
  if (mode == COMM_ALLGATHER_A && a_mn_major) return -6;
  if (!(use_multimem && mc_base != nullptr) && world > 8) return -9;  // peer-load reduction is unrolled for <= 8 ranks
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(nullptr); ctx_bound = true; }
  const bool fp16 = (flags & GEMM_FLAG_FP16) != 0;
  const int bn = wide_tiles ? 256 : 128;
  uint8_t* stage = static_cast<uint8_t*>(own_buf) + data_off;
  GemmParams p;
  p.bias = bias; p.aux = nullptr; p.aux_out = aux_out; p.ld_aux = 0; p.ld_aux_out = ld_aux_out;
  p.M = M; p.N = N; p.K = K; p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major; p.flags = flags; p.alpha = alpha;
  p.err = err_word;
  CommParams& c = p.comm;
  c.peer_bufs = peer_bufs_dev; c.mc_base = static_cast<uint8_t*>(mc_base); c.data_off = data_off; c.flag_off = flag_off;
  c.rank = rank; c.world = world; c.epoch = epoch; c.mode = mode; c.use_multimem = use_multimem && mc_base != nullptr;
  {
    // readiness words of this call must fit below the completion counter, which sits in the last 64 bytes
    const long long tiles = static_cast<long long>((M + BM - 1) / BM) * ((N + bn - 1) / bn);
    const long long words = mode == COMM_ALLGATHER_A ? static_cast<long long>((M + BM - 1) / BM) * 8 * COMM_WARPS
                                                     : tiles * world * 4;
    if (words * 4 > flag_bytes - 64) return -8;
    c.done_off = flag_off + flag_bytes - 64;
    c.done_target = done_base + static_cast<unsigned>(tiles) * COMM_WARPS;
  }
  c.out = out; c.ld_out = ld_out; c.ag_src = nullptr; c.ld_ag_src = 0; c.ag_parts = 1;
  {
    const char* dbg = getenv("OSLO_B200_COMM_DEBUG");
    c.debug = dbg ? atoi(dbg) : 0;
  }
  c.trace = trace;
  CUtensorMap ta, tb;
  int rc;
  if (mode == COMM_ALLGATHER_A) {
    // A (this rank's shard, ordinary memory) is pushed into the gather buffer; the GEMM reads the buffer
    c.ag_src = A; c.ld_ag_src = lda;
    int parts = 1;
    while (parts < 8 && (K / (parts * 2)) % 8 == 0 && (K / (parts * 2)) >= 256) parts *= 2;
    c.ag_parts = parts;
    rc = make_tma_2d_16bit(&ta, stage, K, M, K, BM, fp16);
    p.D = out; p.ldd = ld_out;
  } else {
    if (!a_mn_major) rc = make_tma_2d_16bit(&ta, A, K, M, lda, BM, fp16);
    else rc = make_tma_2d_16bit(&ta, A, M, K, lda, 64, fp16);
    p.D = stage; p.ldd = N;  // partial sums go to this rank's symmetric buffer
    // epilogue math must follow the reduction, not precede it; the one exception is adding another per-rank partial
    // sum (aux, [M, N], input dtype) to this rank's tile before it is reduced, which lets two row-parallel products
    // (attention output projection and fc_out of a parallel block) share one collective
    if (flags & (GEMM_FLAG_BIAS | GEMM_FLAG_GELU | GEMM_FLAG_SAVE_PREACT | GEMM_FLAG_OUT_FP32 | GEMM_FLAG_ACCUMULATE |
                 GEMM_FLAG_DGELU))
      return -7;
    if (flags & GEMM_FLAG_RESIDUAL) {
      if (!aux) return -7;
      p.aux = aux; p.ld_aux = ld_aux;
    }
  }
  if (rc) return rc;
  if (!b_mn_major) rc = make_tma_2d_16bit(&tb, B, K, N, ldb, bn, fp16);
  else rc = make_tma_2d_16bit(&tb, B, N, K, ldb, 64, fp16);
  if (rc) return rc - 1000;
  if (bn == 256) return launch_comm<256, 4>(ta, tb, p, num_sms, stream);
  return launch_comm<128, 6>(ta, tb, p, num_sms, stream);
}
