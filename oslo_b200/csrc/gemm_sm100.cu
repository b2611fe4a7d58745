// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D[M,N] = alpha * sum_k A[m,k] * B[n,k]   (+ bias[n]) (gelu) (* gelu'(aux)) (+ residual) (+ D)
//
// A is stored [M,K] (K-major) or [K,M] (MN-major); B is stored [N,K] (K-major) or [K,N] (MN-major), so
// forward, dgrad and wgrad of a linear layer - in both the nn.Linear [out,in] and the Conv1D [in,out]
// weight layouts - run without any transpose copy: the operand "major" is a bit of the instruction
// descriptor and a different TMA box shape.
//
// Roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = TMEM owner + MMA issuer (one lane),
// warps 2..5 = epilogue (TMEM -> registers -> global). Tiles of 128 x BN x 64 flow through a STAGES-deep
// shared-memory ring guarded by full/empty mbarriers; two TMEM accumulators (2 x BN columns) let the
// epilogue of tile i overlap the main loop of tile i+1. All waits are bounded (ptx.cuh).
#include <mutex>

#include <cstdlib>

#include "gemm_core.cuh"
#include "gemm_pair_core.cuh"

namespace oslo {

// ---------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 2-D map over a row-major [outer, inner] matrix of 16-bit elements with a {64, box_rows} box, 128-B swizzle
int make_tma_2d_16bit(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride_elems,
                      uint32_t box_rows, bool fp16) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -100;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || (row_stride_elems * 2) % 16) return -101;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(1000 + static_cast<int>(r));
}

// N-D (rank 3..5) map over 16-bit elements; dim 0 is contiguous, `strides_elems[i]` is the element stride of
// dim i + 1; the box is `box[]` elements per dim, 128-B swizzle (so box[0] must be 64), zero fill out of range
int make_tma_nd_16bit(CUtensorMap* map, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_elems,
                      const uint32_t* box, bool fp16) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -100;
  if (rank < 2 || rank > 5 || (reinterpret_cast<uintptr_t>(ptr) & 15)) return -101;
  cuuint64_t d[5], st[4];
  cuuint32_t bx[5], estr[5];
  for (int i = 0; i < rank; ++i) { d[i] = dims[i]; bx[i] = box[i]; estr[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) {
    st[i] = strides_elems[i] * 2;
    if (st[i] % 16) return -101;
  }
  CUresult r = enc(map, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank,
                   const_cast<void*>(ptr), d, st, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(1000 + static_cast<int>(r));
}

template <int BN, int STAGES>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int num_sms, cudaStream_t stream);

// Few-row GEMM (decode steps): 128 x 128 tiles whose k range is cut into `split_k` slices so that all SMs stream
// weights; slice s writes its partial sums to plane s of the fp32 workspace D [split_k, M, N].
static int launch_split_k(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int split_k, int num_sms,
                          cudaStream_t stream) {
  p.split_k = split_k;
  return launch<128, 6>(ta, tb, p, num_sms, stream);
}

template <int BN, int STAGES>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int num_sms, cudaStream_t stream) {
  constexpr size_t smem = STAGES * (BM * BK * 2 + BN * BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n * p.split_k;
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_tcgen05_kernel<BN, STAGES, false><<<grid, GEMM_THREADS, smem, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

constexpr int PAIR_STAGES = 6;   // 32 KB operand stages; OSLO_B200_PAIR_STAGES=7 fills the 227 KB (no measurable gain: the part is power-bound)

// 256 x 256 tiles on CTA pairs (gemm_pair_core.cuh); the grid is a whole number of pairs
template <int STAGES>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int num_sms, cudaStream_t stream) {
  constexpr size_t smem = STAGES * (2 * BM * BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
  static_assert(smem <= 232448, "shared memory budget of one CTA");
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_tcgen05_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  p.tiles_m = (p.M + PAIR_TILE - 1) / PAIR_TILE;
  p.tiles_n = (p.N + PAIR_TILE - 1) / PAIR_TILE;
  static const int group_m = [] { const char* e = getenv("OSLO_B200_GEMM_GROUP_M"); const int v = e ? atoi(e) : 8; return v > 0 ? v : 8; }();
  p.group_m = group_m;
  const int tiles = p.tiles_m * p.tiles_n;
  // persistent kernel: no more pairs than can be resident at once (pairs are placed as clusters of two SMs)
  static int max_pairs = 0;
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(num_sms / 2 * 2));
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_tcgen05_kernel<STAGES>, &cfg) != cudaSuccess || n <= 0) n = num_sms / 2;
    max_pairs = n;
  }
  const int pairs = std::min(tiles, std::min(max_pairs, num_sms / 2));   // num_sms already excludes reserved SMs
  gemm_pair_tcgen05_kernel<STAGES><<<2 * pairs, GEMM_THREADS, smem, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

// 0 = single-CTA tiles only (OSLO_B200_GEMM_PAIR=0), 1 = CTA pairs for large outputs (default)
static bool pair_enabled() {
  static const bool on = [] { const char* e = getenv("OSLO_B200_GEMM_PAIR"); return !(e && e[0] == '0'); }();
  return on;
}

// Tile shape selection, tensor maps and launch for a filled-in GemmParams (M, N, K, majors, flags, epilogue operands)
static int dispatch_gemm(const void* A, const void* B, int lda, int ldb, GemmParams& p, int num_sms, cudaStream_t stream);

}  // namespace oslo

extern "C" int oslo_gemm_16bit(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb, int ldd,
                               int a_mn_major, int b_mn_major, const void* bias, const void* aux, int ld_aux,
                               void* aux_out, int ld_aux_out, int flags, float alpha, int* err_word, int num_sms,
                               cudaStream_t stream) {
  using namespace oslo;
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if (flags & (GEMM_FLAG_CE_STATS | GEMM_FLAG_CE_GRAD)) return -7;   // those epilogues come through oslo_gemm_ce_16bit
  GemmParams p;
  p.D = D; p.bias = bias; p.aux = aux; p.aux_out = aux_out;
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ld_aux = ld_aux; p.ld_aux_out = ld_aux_out;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major; p.flags = flags; p.alpha = alpha; p.err = err_word;
  p.comm = CommParams{};
  return dispatch_gemm(A, B, lda, ldb, p, num_sms, stream);
}

extern "C" int oslo_gemm_ce_16bit(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int b_mn_major,
                                  const void* bias, const long long* labels, long long vocab_start, int mode,
                                  float* stats, const float* lse, const float* scale, void* D, int ldd, int fp16,
                                  int* err_word, int num_sms, cudaStream_t stream) {
  using namespace oslo;
  if (M <= 0 || N <= 0 || K <= 0 || labels == nullptr) return -1;
  if (mode == 0 ? stats == nullptr : (lse == nullptr || scale == nullptr || D == nullptr)) return -1;
  GemmParams p;
  p.D = D; p.bias = bias; p.aux = nullptr; p.aux_out = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ld_aux = 0; p.ld_aux_out = 0;
  p.a_mn_major = 0; p.b_mn_major = b_mn_major; p.alpha = 1.f; p.err = err_word;
  p.flags = (mode == 0 ? GEMM_FLAG_CE_STATS : GEMM_FLAG_CE_GRAD) | (bias ? GEMM_FLAG_BIAS : 0) | (fp16 ? GEMM_FLAG_FP16 : 0);
  p.ce_labels = labels; p.ce_vocab_start = vocab_start; p.ce_stats = stats; p.ce_lse = lse; p.ce_scale = scale;
  p.comm = CommParams{};
  return dispatch_gemm(A, B, lda, ldb, p, num_sms, stream);
}

namespace oslo {
static int dispatch_gemm(const void* A, const void* B, int lda, int ldb, GemmParams& p, int num_sms, cudaStream_t stream) {
  const int M = p.M, N = p.N, K = p.K, a_mn_major = p.a_mn_major, b_mn_major = p.b_mn_major, flags = p.flags;
  // the tensor-map encoder is a driver-API call and needs the primary context bound to THIS thread; the
  // autograd engine's worker threads may not have made a runtime call yet
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(nullptr); ctx_bound = true; }
  const bool fp16 = (flags & GEMM_FLAG_FP16) != 0;
  // narrow outputs use the 128-wide tile so that more CTAs share the work
  const bool wide = (N >= 256) && (static_cast<long long>((M + BM - 1) / BM) * ((N + 255) / 256) >= num_sms / 2);
  // large outputs: 256 x 256 tiles on CTA pairs, when they fill the pairs at least as well as single tiles fill the SMs
  const long long pair_tiles = static_cast<long long>((M + PAIR_TILE - 1) / PAIR_TILE) * ((N + PAIR_TILE - 1) / PAIR_TILE);
  const bool pair = pair_enabled() && wide && M >= PAIR_TILE && pair_tiles >= num_sms / 2;
  const int bn = pair ? BM : (wide ? 256 : 128);   // B box rows: a pair's CTA stages 128 of the 256 tile columns
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn_major) rc = make_tma_2d_16bit(&ta, A, K, M, lda, BM, fp16);
  else rc = make_tma_2d_16bit(&ta, A, M, K, lda, 64, fp16);
  if (rc) return rc;  // -(1000 + CUresult): encoding the A map failed
  if (!b_mn_major) rc = make_tma_2d_16bit(&tb, B, K, N, ldb, bn, fp16);
  else rc = make_tma_2d_16bit(&tb, B, N, K, ldb, 64, fp16);
  if (rc) return rc - 1000;  // -(2000 + CUresult): encoding the B map failed
  if (pair) {
    static const int stages = [] { const char* e = getenv("OSLO_B200_PAIR_STAGES"); return e ? atoi(e) : PAIR_STAGES; }();
    if (stages == 7) return launch_pair<7>(ta, tb, p, num_sms, stream);
    return launch_pair<PAIR_STAGES>(ta, tb, p, num_sms, stream);
  }
  if (bn == 256) return launch<256, 4>(ta, tb, p, num_sms, stream);
  return launch<128, 6>(ta, tb, p, num_sms, stream);
}
}  // namespace oslo

// how many k slices a few-row GEMM should use so that about two work items exist per SM (1 = do not split)
extern "C" int oslo_gemm_split_k_for(int M, int N, int K, int num_sms) {
  using namespace oslo;
  if (M > BM) return 1;
  const int tiles = (N + 127) / 128;
  const int kblocks = (K + BK - 1) / BK;
  int s = (2 * num_sms) / (tiles > 0 ? tiles : 1);
  if (s > kblocks / 2) s = kblocks / 2;
  return s < 2 ? 1 : s;
}

// D[s, M, N] (fp32) = partial A B^T of k slice s, for s < split_k; M <= 128. The planes need no initialisation.
extern "C" int oslo_gemm_splitk_16bit(const void* A, const void* B, float* D, int M, int N, int K, int lda, int ldb,
                                      int ldd, int a_mn_major, int b_mn_major, int fp16, int split_k, int* err_word,
                                      int num_sms, cudaStream_t stream) {
  using namespace oslo;
  if (M <= 0 || N <= 0 || K <= 0 || M > BM || split_k < 1 || split_k > (K + BK - 1) / BK) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(nullptr); ctx_bound = true; }
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn_major) rc = make_tma_2d_16bit(&ta, A, K, M, lda, BM, fp16 != 0);
  else rc = make_tma_2d_16bit(&ta, A, M, K, lda, 64, fp16 != 0);
  if (rc) return rc;
  if (!b_mn_major) rc = make_tma_2d_16bit(&tb, B, K, N, ldb, 128, fp16 != 0);
  else rc = make_tma_2d_16bit(&tb, B, N, K, ldb, 64, fp16 != 0);
  if (rc) return rc - 1000;
  GemmParams p;
  p.D = D; p.bias = nullptr; p.aux = nullptr; p.aux_out = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ld_aux = 0; p.ld_aux_out = 0;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.flags = GEMM_FLAG_OUT_FP32 | (fp16 ? GEMM_FLAG_FP16 : 0); p.alpha = 1.f; p.err = err_word;
  p.comm = CommParams{};
  return launch_split_k(ta, tb, p, split_k, num_sms, stream);
}
