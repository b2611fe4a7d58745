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
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "oslo_kernels.h"
#include "ptx.cuh"

namespace oslo {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  void* D;
  const void* bias;     // [N] same dtype as inputs, or nullptr
  const void* aux;      // residual (out dtype, [M,N]) or pre-activation for dgelu (input dtype, [M,N])
  void* aux_out;        // pre-activation output for FLAG_SAVE_PREACT (input dtype, [M,N])
  int M, N, K;
  int ldd, ld_aux, ld_aux_out;
  int a_mn_major, b_mn_major;
  int flags;
  float alpha;
  int* err;
  int tiles_m, tiles_n;
};

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * x * (1.0f + t);
}
__device__ __forceinline__ float dgelu_tanh_f(float x) {
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
  return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * 0.7978845608028654f * (1.0f + 0.134145f * x * x);
}

__device__ __forceinline__ float ld_half_as_float(const void* p, size_t idx, bool fp16) {
  return fp16 ? __half2float(reinterpret_cast<const __half*>(p)[idx])
              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx]);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, bool fp16) {
  if (fp16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void unpack8(const uint4& v, float* f, bool fp16) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (fp16) {
      float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    } else {
      float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
  }
}

// grouped raster: walk GROUP_M row-blocks per column sweep so concurrently running CTAs share B tiles in L2
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GROUP_M = 8;
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const GemmParams p) {
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512, both powers of two >= 32

  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: required by the 128-byte swizzle atoms the descriptors assume
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  // bars: [0,STAGES) full, [STAGES,2S) empty, [2S,2S+2) tmem_full, [2S+2,2S+4) tmem_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
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
      mbar_init(tempty_bar(b), 4);  // one arrival per epilogue warp
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

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, p.err, ERR_WAIT_EMPTY);
          if (!ok) break;
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_2d(sa, &tma_a, full_bar(stage), k0, m0);           // box {64 k, 128 rows}
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)                            // boxes {64 m, 64 k rows}
              tma_load_2d(sa + c * 8192, &tma_a, full_bar(stage), m0 + c * 64, k0);
          }
          if (!p.b_mn_major) {
            tma_load_2d(sb, &tma_b, full_bar(stage), k0, n0);           // box {64 k, BN rows}
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sb + c * 8192, &tma_b, full_bar(stage), n0 + c * 64, k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const int fmt = (p.flags & GEMM_FLAG_FP16) ? 0 : 1;
      const uint32_t idesc = make_idesc_f16(BM, BN, fmt, p.a_mn_major, p.b_mn_major);
      // K-major tile: rows of 128 B, 8-row groups 1024 B apart, one k-step (16 elements) = 32 B
      // MN-major tile: k rows of 128 B, 64-wide MN chunks 8192 B apart, one k-step (16 rows) = 2048 B
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, a_step = p.a_mn_major ? 2048u : 32u;
      const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u, b_step = p.b_mn_major ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        ok = mbar_wait(tempty_bar(buf), acc_phase[buf] ^ 1, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        acc_phase[buf] ^= 1;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * BN;
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
            umma_f16(tmem_acc, da, db, idesc, (kb | k) != 0);
          }
          umma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(tfull_bar(buf));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const bool fp16 = (p.flags & GEMM_FLAG_FP16) != 0;
    const bool out_f32 = (p.flags & GEMM_FLAG_OUT_FP32) != 0;
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      int tm, tn;
      tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
      ok = mbar_wait(tfull_bar(buf), acc_phase[buf], abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      acc_phase[buf] ^= 1;
      tc_fence_after();
      const int row = tm * BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_wait_ld();
        const int col0 = tn * BN + c0;
        if (!row_ok || col0 >= p.N) continue;
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
        const int ncols = min(32, p.N - col0);
        const bool vec = (ncols == 32);
        if (p.flags & GEMM_FLAG_BIAS) {
          if (vec) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              float b[8];
              unpack8(*reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.bias) + col0 + i), b, fp16);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[i + j] += b[j];
            }
          } else {
            _Pragma("unroll") for (int i = 0; i < 32; ++i) if (i < ncols) v[i] += ld_half_as_float(p.bias, col0 + i, fp16);
          }
        }
        if (p.flags & GEMM_FLAG_SAVE_PREACT) {
          uint16_t* z = reinterpret_cast<uint16_t*>(p.aux_out) + static_cast<size_t>(row) * p.ld_aux_out + col0;
          if (vec) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 o;
              o.x = pack2(v[i], v[i + 1], fp16); o.y = pack2(v[i + 2], v[i + 3], fp16);
              o.z = pack2(v[i + 4], v[i + 5], fp16); o.w = pack2(v[i + 6], v[i + 7], fp16);
              *reinterpret_cast<uint4*>(z + i) = o;
            }
          } else {
            _Pragma("unroll") for (int i = 0; i < 32; ++i) if (i < ncols) z[i] = static_cast<uint16_t>(pack2(v[i], 0.f, fp16) & 0xffff);
          }
        }
        if (p.flags & GEMM_FLAG_GELU) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_f(v[i]);
        }
        if (p.flags & GEMM_FLAG_DGELU) {
          const uint16_t* z = reinterpret_cast<const uint16_t*>(p.aux) + static_cast<size_t>(row) * p.ld_aux + col0;
          if (vec) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              float zz[8];
              unpack8(*reinterpret_cast<const uint4*>(z + i), zz, fp16);
#pragma unroll
              for (int j = 0; j < 8; ++j) v[i + j] *= dgelu_tanh_f(zz[j]);
            }
          } else {
            _Pragma("unroll") for (int i = 0; i < 32; ++i) if (i < ncols) v[i] *= dgelu_tanh_f(ld_half_as_float(z, i, fp16));
          }
        }
        if (p.flags & GEMM_FLAG_RESIDUAL) {
          if (out_f32) {
            const float* rr = reinterpret_cast<const float*>(p.aux) + static_cast<size_t>(row) * p.ld_aux + col0;
            _Pragma("unroll") for (int i = 0; i < 32; ++i) if (i < ncols) v[i] += rr[i];
          } else {
            const uint16_t* rr = reinterpret_cast<const uint16_t*>(p.aux) + static_cast<size_t>(row) * p.ld_aux + col0;
            if (vec) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                float x[8];
                unpack8(*reinterpret_cast<const uint4*>(rr + i), x, fp16);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i + j] += x[j];
              }
            } else {
              _Pragma("unroll") for (int i = 0; i < 32; ++i) if (i < ncols) v[i] += ld_half_as_float(rr, i, fp16);
            }
          }
        }
        if (out_f32) {
          float* d = reinterpret_cast<float*>(p.D) + static_cast<size_t>(row) * p.ldd + col0;
          if (vec) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
              if (p.flags & GEMM_FLAG_ACCUMULATE) {
                const float4 old = *reinterpret_cast<const float4*>(d + i);
                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
              }
              *reinterpret_cast<float4*>(d + i) = o;
            }
          } else {
            _Pragma("unroll") for (int i = 0; i < 32; ++i) if (i < ncols) d[i] = v[i] + ((p.flags & GEMM_FLAG_ACCUMULATE) ? d[i] : 0.f);
          }
        } else {
          uint16_t* d = reinterpret_cast<uint16_t*>(p.D) + static_cast<size_t>(row) * p.ldd + col0;
          if (vec) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (p.flags & GEMM_FLAG_ACCUMULATE) {
                float x[8];
                unpack8(*reinterpret_cast<const uint4*>(d + i), x, fp16);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[i + j] += x[j];
              }
              uint4 o;
              o.x = pack2(v[i], v[i + 1], fp16); o.y = pack2(v[i + 2], v[i + 3], fp16);
              o.z = pack2(v[i + 4], v[i + 5], fp16); o.w = pack2(v[i + 6], v[i + 7], fp16);
              *reinterpret_cast<uint4*>(d + i) = o;
            }
          } else {
            _Pragma("unroll") for (int i = 0; i < 32; ++i) if (i < ncols) {
              float x = v[i];
              if (p.flags & GEMM_FLAG_ACCUMULATE) x += ld_half_as_float(d, i, fp16);
              d[i] = static_cast<uint16_t>(pack2(x, 0.f, fp16) & 0xffff);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
  }

  // ------------------------------------------------------------ teardown
  if (*abort_flag) {
    // give copies that are still in flight time to land before shared memory is released
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

template <int BN, int STAGES>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams& p, int num_sms, cudaStream_t stream) {
  constexpr size_t smem = STAGES * (BM * BK * 2 + BN * BK * 2) + (2 * STAGES + 4) * 8 + 16 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  p.tiles_m = (p.M + BM - 1) / BM;
  p.tiles_n = (p.N + BN - 1) / BN;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < num_sms ? tiles : num_sms;
  gemm_tcgen05_kernel<BN, STAGES><<<grid, GEMM_THREADS, smem, stream>>>(ta, tb, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace oslo

extern "C" int oslo_gemm_16bit(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb, int ldd,
                               int a_mn_major, int b_mn_major, const void* bias, const void* aux, int ld_aux,
                               void* aux_out, int ld_aux_out, int flags, float alpha, int* err_word, int num_sms,
                               cudaStream_t stream) {
  using namespace oslo;
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  // the tensor-map encoder is a driver-API call and needs the primary context bound to THIS thread; the
  // autograd engine's worker threads may not have made a runtime call yet
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(nullptr); ctx_bound = true; }
  const bool fp16 = (flags & GEMM_FLAG_FP16) != 0;
  // narrow outputs use the 128-wide tile so that more CTAs share the work
  const bool wide = (N >= 256) && (static_cast<long long>((M + BM - 1) / BM) * ((N + 255) / 256) >= num_sms / 2);
  const int bn = wide ? 256 : 128;
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn_major) rc = make_tma_2d_16bit(&ta, A, K, M, lda, BM, fp16);
  else rc = make_tma_2d_16bit(&ta, A, M, K, lda, 64, fp16);
  if (rc) return rc;  // -(1000 + CUresult): encoding the A map failed
  if (!b_mn_major) rc = make_tma_2d_16bit(&tb, B, K, N, ldb, bn, fp16);
  else rc = make_tma_2d_16bit(&tb, B, N, K, ldb, 64, fp16);
  if (rc) return rc - 1000;  // -(2000 + CUresult): encoding the B map failed
  GemmParams p;
  p.D = D; p.bias = bias; p.aux = aux; p.aux_out = aux_out;
  p.M = M; p.N = N; p.K = K; p.ldd = ldd; p.ld_aux = ld_aux; p.ld_aux_out = ld_aux_out;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major; p.flags = flags; p.alpha = alpha; p.err = err_word;
  if (bn == 256) return launch<256, 4>(ta, tb, p, num_sms, stream);
  return launch<128, 6>(ta, tb, p, num_sms, stream);
}
