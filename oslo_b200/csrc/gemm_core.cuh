// tcgen05 GEMM core shared by the plain GEMM (gemm_sm100.cu) and the GEMM + collective kernels
// (fused_comm_gemm.cu). See gemm_sm100.cu for the operand conventions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "oslo_kernels.h"
#include "ptx.cuh"

namespace oslo {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

// Collective fused into the GEMM (all addresses are byte offsets into the symmetric buffer of the group).
enum : int { COMM_NONE = 0, COMM_ALLREDUCE = 1, COMM_REDUCE_SCATTER = 2, COMM_ALLGATHER_A = 3 };
struct CommParams {
  void* const* peer_bufs;  // device array [world]: peer-mapped base address of every rank's symmetric buffer
  uint8_t* mc_base;        // NVSwitch multicast mapping of the same buffer, or nullptr
  long long data_off;      // staging matrix: partial outputs [M,N] (reduce modes) or gathered A [M,K] (all-gather)
  long long flag_off;      // uint32 flags: one per tile / chunk, then the completion counter
  int rank, world;
  uint32_t epoch;          // generation of this call on its workspace slot (1, 2, 3, ...). Readiness words are
                           // WRITTEN with this value (never counted), so stale words of earlier calls - whatever
                           // their shape or mode - are simply smaller and nothing ever needs a reset
  long long done_off;      // all-reduce: byte offset of the completion counter (counted; fixed location per slot)
  uint32_t done_target;    // value the completion counter reaches when every tile of this call is final
  int mode;
  int use_multimem;
  void* out;               // reduce-scatter: this rank's [M/world, N] result (ordinary memory)
  int ld_out;
  const void* ag_src;      // all-gather: this rank's [M/world, K] shard (ordinary memory)
  int ld_ag_src;
  int ag_parts;            // column parts per 128-row chunk
  unsigned long long* trace;  // optional [gridDim.x][8] device timestamps (ns) of the phases of every CTA, or nullptr
  int debug;               // experiments: bit 0 = gpu-scope fence in the epilogue, bit 1 = communication warps move no data
};

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
  int group_m = 8;      // row blocks per column sweep of the tile raster
  int split_k = 1;      // > 1: every tile's k range is cut into this many work items; slice s writes its fp32 partial
                        // result to plane s of D ([split_k, M, ldd] fp32); other epilogue flags are ignored
  // cross-entropy epilogues (GEMM_FLAG_CE_STATS / GEMM_FLAG_CE_GRAD)
  const long long* ce_labels = nullptr;   // [M] global vocabulary ids
  long long ce_vocab_start = 0;           // id of this matrix's column 0
  float* ce_stats = nullptr;              // [ceil(N / 128), M, 3]
  const float* ce_lse = nullptr;          // [M]
  const float* ce_scale = nullptr;        // [M]
  CommParams comm;
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
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn, int GROUP_M = 8) {
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % rows;
  tn = r / rows;
}

constexpr int COMM_WARPS = 8;
constexpr int COMM_THREADS = 32 * COMM_WARPS;
constexpr int GEMM_THREADS_COMM = GEMM_THREADS + 32 * COMM_WARPS;

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_red_release_add(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 mm_ld_reduce_16(const void* mc, bool fp16) {
  uint4 v;
  if (fp16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_16(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w) : "memory");
}
// wait until *flag has reached `target` (flags only grow; compare as a signed distance so wrap-around is harmless)
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t target, volatile int* abort_flag,
                                             int* err_word) {
  if (static_cast<int32_t>(ld_acquire_sys(flag) - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (static_cast<int32_t>(ld_acquire_sys(flag) - target) < 0) {
    if ((++spins & 0x3f) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > OSLO_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (err_word) atomicCAS(err_word, 0, ERR_WAIT_PEER);
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_red_release_max(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.max.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
// Whole-warp wait: words[0 .. nwords) must all have reached generation `gen` (lanes stride over the words).
// Returns the same value on every lane.
__device__ __forceinline__ bool warp_wait_words(const uint32_t* words, int nwords, uint32_t gen,
                                                volatile int* abort_flag, int* err_word) {
  const int lane = threadIdx.x & 31;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    bool mine = true;
    for (int i = lane; i < nwords; i += 32) mine = mine && (static_cast<int32_t>(ld_acquire_sys(words + i) - gen) >= 0);
    if (__all_sync(0xffffffffu, mine)) return true;
    __nanosleep(100);  // keep the polling traffic of idle communication warps off the L2
    if ((++spins & 0x3f) == 0) {
      bool give_up = (*abort_flag != 0);
      if (!give_up && globaltimer_ns() - t0 > OSLO_WAIT_LIMIT_NS) {
        give_up = true;
        *abort_flag = 1;
        if (err_word) atomicCAS(err_word, 0, ERR_WAIT_PEER);
      }
      if (__any_sync(0xffffffffu, give_up)) return false;
    }
  }
}

// Readiness words and ownership are indexed by idx = tm * tiles_n + tn.
// all-reduce: owner = idx % world (work spread evenly); reduce-scatter: the rank that keeps row block tm.
__device__ __forceinline__ int tile_owner(const CommParams& c, int idx, int tm, int tiles_m) {
  if (c.mode == COMM_REDUCE_SCATTER) return tm / (tiles_m / c.world);
  return idx % c.world;
}

// Cross-entropy statistics of one row, accumulated over the 32-column chunks of a 128-column block in the epilogue:
// running max, sum of exp(x - max) and the logit of the row's label when it lies in the block (x = acc + bias).
struct CeAcc {
  float m, s, t;
};
__device__ __forceinline__ void ce_reset(CeAcc& a) { a.m = -3.0e38f; a.s = 0.f; a.t = 0.f; }
__device__ __forceinline__ void ce_accumulate(const GemmParams& p, int col0, const uint32_t (&r)[32], bool fp16,
                                              long long label_local, CeAcc& a) {
  float v[32];
  const int ncols = min(32, p.N - col0);
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
  if (p.flags & GEMM_FLAG_BIAS) {
    if (ncols == 32) {
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
  // the loss is defined on the 16-bit logits a separate GEMM would have written: round as that store would
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const uint32_t pk = pack2(v[i], v[i + 1], fp16);
    if (fp16) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pk));
      v[i] = f.x; v[i + 1] = f.y;
    } else {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk));
      v[i] = f.x; v[i + 1] = f.y;
    }
  }
  float mx = a.m;
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (i < ncols) mx = fmaxf(mx, v[i]);
  float s = a.s * exp2f((a.m - mx) * 1.4426950408889634f);
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (i < ncols) s += exp2f((v[i] - mx) * 1.4426950408889634f);
  a.m = mx;
  a.s = s;
  const long long d = label_local - col0;
  if (d >= 0 && d < ncols) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i == d) a.t = v[i];
  }
}
// one record per (128-column block, row); written after the block's last chunk that holds valid columns
__device__ __forceinline__ void ce_flush_if_block_ends(const GemmParams& p, int row, int col0, CeAcc& a) {
  const bool last_chunk_of_block = ((col0 + 32) % GEMM_CE_BLOCK) == 0 || col0 + 32 >= p.N;
  if (!last_chunk_of_block) return;
  float* rec = p.ce_stats + (static_cast<size_t>(col0 / GEMM_CE_BLOCK) * p.M + row) * 3;
  rec[0] = a.m; rec[1] = a.s; rec[2] = a.t;
  ce_reset(a);
}

// Epilogue of one [1 row x 32 columns] accumulator chunk held by a thread: alpha, bias, GeLU (+ saved
// pre-activation), dGeLU, residual, accumulate, conversion and the store. `row` < M and `col0` < N are the
// caller's responsibility.
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, int row, int col0, const uint32_t (&r)[32],
                                               bool fp16, bool out_f32, int kslice = 0) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
    const int ncols = min(32, p.N - col0);
    if (p.split_k > 1) {  // partial sums of k slice `kslice` go to their own [M, ldd] fp32 plane (deterministic)
      float* d = reinterpret_cast<float*>(p.D) + (static_cast<size_t>(kslice) * p.M + row) * p.ldd + col0;
      if (ncols == 32) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(d + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < ncols) d[i] = v[i];
      }
      return;
    }
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
    if (p.flags & GEMM_FLAG_CE_GRAD) {
      // (softmax - onehot) * scale of the recomputed logits (rounded to the 16-bit value the forward pass used)
      const float l = p.ce_lse[row], sc = p.ce_scale[row];
      const long long d = p.ce_labels[row] - p.ce_vocab_start - col0;
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const uint32_t pk = pack2(v[i], v[i + 1], fp16);
        float2 f;
        if (fp16) f = __half22float2(*reinterpret_cast<const __half2*>(&pk));
        else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk));
        v[i] = exp2f((f.x - l) * 1.4426950408889634f);
        v[i + 1] = exp2f((f.y - l) * 1.4426950408889634f);
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (i == d) v[i] -= 1.f;
        v[i] *= sc;
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

template <int BN, int STAGES, bool COMM>
__global__ void __launch_bounds__(COMM ? GEMM_THREADS_COMM : GEMM_THREADS, 1)
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
  unsigned long long* trace = nullptr;
  if (COMM && p.comm.trace) {
    trace = p.comm.trace + static_cast<size_t>(blockIdx.x) * 8;
    if (threadIdx.x == 0) trace[0] = globaltimer_ns();
  }

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;
  // work item = (tile, k slice); one slice per tile unless split_k > 1
  const int split_k = COMM ? 1 : p.split_k;
  const int num_items = num_tiles * split_k;
  // all-gather mode walks the row blocks starting with this rank's own shard, which needs no transfer
  auto coords = [&](int tile, int& tm, int& tn) {
    tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
    if (COMM && p.comm.mode == COMM_ALLGATHER_A) {
      tm += p.comm.rank * (p.tiles_m / p.comm.world);
      if (tm >= p.tiles_m) tm -= p.tiles_m;
    }
    if (COMM && p.comm.mode == COMM_REDUCE_SCATTER) {
      // interleave the ranks' row blocks in time: raster position i -> block (i / world) of rank (i % world)
      const int per = p.tiles_m / p.comm.world;
      tm = (tm % p.comm.world) * per + tm / p.comm.world;
    }
  };

  if (COMM && warp == 0 && p.comm.mode == COMM_ALLGATHER_A) {
    // ------------------------------------------------------------ TMA producer, all-gather mode: the whole warp
    // waits for the row block to arrive from its source rank, lane 0 issues the copies
    const uint32_t* words = reinterpret_cast<const uint32_t*>(
        static_cast<const uint8_t*>(p.comm.peer_bufs[p.comm.rank]) + p.comm.flag_off);
    const int nwords = p.comm.ag_parts * COMM_WARPS;
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int tm, tn;
      coords(tile, tm, tn);
      const int m0 = tm * BM, n0 = tn * BN;
      ok = warp_wait_words(words + static_cast<size_t>(tm) * nwords, nwords, p.comm.epoch, abort_flag, p.err);
      if (!ok) break;
      asm volatile("fence.proxy.async.global;" ::: "memory");  // the TMA engine reads what peers just wrote
      for (int kb = 0; kb < kblocks; ++kb) {
        int ok_l = 1;
        if (lane == 0) {
          ok_l = mbar_wait(empty_bar(stage), phase ^ 1, abort_flag, p.err, ERR_WAIT_EMPTY) ? 1 : 0;
          if (ok_l) {
            const uint32_t sa = smem_base + stage * STAGE_BYTES;
            const uint32_t sb = sa + A_BYTES;
            mbar_expect_tx(full_bar(stage), STAGE_BYTES);
            const int k0 = kb * BK;
            tma_load_2d(sa, &tma_a, full_bar(stage), k0, m0);
            if (!p.b_mn_major) {
              tma_load_2d(sb, &tma_b, full_bar(stage), k0, n0);
            } else {
#pragma unroll
              for (int c = 0; c < BN / 64; ++c)
                tma_load_2d(sb + c * 8192, &tma_b, full_bar(stage), n0 + c * 64, k0);
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok_l, 0) != 0;
        if (!ok) break;
        if (++stage == STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tma_a);
      tma_prefetch_desc(&tma_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int tile = item % num_tiles, ks = item / num_tiles;
        const int kb0 = ks * kblocks / split_k, kb1 = (ks + 1) * kblocks / split_k;
        int tm, tn;
        coords(tile, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
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
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++local) {
        const int ks = item / num_tiles;
        const int kb0 = ks * kblocks / split_k, kb1 = (ks + 1) * kblocks / split_k;
        const int buf = local & 1;
        ok = mbar_wait(tempty_bar(buf), acc_phase[buf] ^ 1, abort_flag, p.err, ERR_WAIT_TMEM_EMPTY);
        if (!ok) break;
        acc_phase[buf] ^= 1;
        tc_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          ok = mbar_wait(full_bar(stage), phase, abort_flag, p.err, ERR_WAIT_FULL);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = make_smem_desc(sa + k * a_step, a_lbo, 1024);
            const uint64_t db = make_smem_desc(sb + k * b_step, b_lbo, 1024);
            umma_f16(tmem_acc, da, db, idesc, (kb != kb0) || (k != 0));
          }
          umma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(tfull_bar(buf));
      }
      if (trace) trace[2] = globaltimer_ns();
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const bool fp16 = (p.flags & GEMM_FLAG_FP16) != 0;
    const bool out_f32 = (p.flags & GEMM_FLAG_OUT_FP32) != 0;
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++local) {
      const int tile = item % num_tiles, kslice = item / num_tiles;
      const int buf = local & 1;
      int tm, tn;
      coords(tile, tm, tn);
      ok = mbar_wait(tfull_bar(buf), acc_phase[buf], abort_flag, p.err, ERR_WAIT_TMEM_FULL);
      if (!ok) break;
      acc_phase[buf] ^= 1;
      tc_fence_after();
      const int row = tm * BM + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * BN;
      const bool ce_stats = !COMM && (p.flags & GEMM_FLAG_CE_STATS);
      CeAcc ce;
      ce_reset(ce);
      const long long label_local = (ce_stats && row_ok) ? p.ce_labels[row] - p.ce_vocab_start : -1;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_wait_ld();
        const int col0 = tn * BN + c0;
        if (!row_ok || col0 >= p.N) continue;
        if (ce_stats) {
          ce_accumulate(p, col0, r, fp16, label_local, ce);
          ce_flush_if_block_ends(p, row, col0, ce);
        } else {
          epilogue_chunk(p, row, col0, r, fp16, out_f32, kslice);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
      if (COMM && (p.comm.mode == COMM_ALLREDUCE || p.comm.mode == COMM_REDUCE_SCATTER)) {
        // this rank's partial tile is in its symmetric buffer: publish it to the rank that reduces the tile
        // (one word per (tile, rank, epilogue warp), so no CTA-wide barrier and no counting is needed)
        // warp barrier orders the lanes' stores before lane 0's release at system scope (one fence per warp, not 32)
        __syncwarp();
        if (lane == 0) {
          const uint64_t tf0 = trace ? globaltimer_ns() : 0;
          if (p.comm.debug & 1) __threadfence(); else __threadfence_system();
          if (trace && warp == 2) trace[5] += globaltimer_ns() - tf0;
          const int idx = tm * p.tiles_n + tn;
          const int owner = tile_owner(p.comm, idx, tm, p.tiles_m);
          uint32_t* f = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(p.comm.peer_bufs[owner]) + p.comm.flag_off) +
                        (static_cast<size_t>(idx) * p.comm.world + p.comm.rank) * 4 + (warp - 2);
          if (p.comm.debug & 1) *reinterpret_cast<volatile uint32_t*>(f) = p.comm.epoch; else st_release_sys(f, p.comm.epoch);
        }
      }
    }
    if (trace && warp == 2 && lane == 0) trace[3] = globaltimer_ns();
  } else if (COMM) {
    // ------------------------------------------------------------ communication warps (6 ..)
    const CommParams& c = p.comm;
    const int cw = threadIdx.x - GEMM_THREADS;  // 0 .. COMM_THREADS-1
    const bool fp16 = (p.flags & GEMM_FLAG_FP16) != 0;
    uint8_t* my_base = static_cast<uint8_t*>(c.peer_bufs[c.rank]);
    uint32_t* my_flags = reinterpret_cast<uint32_t*>(my_base + c.flag_off);
    const bool mm = c.use_multimem && c.mc_base != nullptr;
    bool ok = true;
    if (c.mode == COMM_ALLGATHER_A) {
      // push this rank's [M/world, K] shard into every rank's gather buffer, 128-row chunk by chunk
      const int rows_per_rank = p.M / c.world;
      const int chunks = rows_per_rank / BM;
      const int parts = c.ag_parts;
      const int cols_per_part = p.K / parts;  // multiple of 8
      const int vpr = cols_per_part / 8;
      const uint16_t* src = reinterpret_cast<const uint16_t*>(c.ag_src);
      for (int unit = blockIdx.x; unit < chunks * parts; unit += gridDim.x) {
        const int ch = unit / parts, part = unit % parts;
        const int total = BM * vpr;
        for (int base = cw; base < total; base += COMM_THREADS * 4) {
          uint4 val[4];
          size_t off[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int idx = base + j * COMM_THREADS;
            if (idx < total) {
              const int r = idx / vpr, v = idx % vpr;
              const int col = part * cols_per_part + v * 8;
              val[j] = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(ch * BM + r) * c.ld_ag_src + col);
              off[j] = c.data_off + (static_cast<size_t>(c.rank * rows_per_rank + ch * BM + r) * p.K + col) * 2;
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (base + j * COMM_THREADS < total) {
              if (mm) {
                mm_st_16(c.mc_base + off[j], val[j]);
              } else {
                for (int w = 0; w < c.world; ++w)
                  *reinterpret_cast<uint4*>(static_cast<uint8_t*>(c.peer_bufs[w]) + off[j]) = val[j];
              }
            }
          }
        }
        __syncwarp();
        if ((cw & 31) == 0) {  // one word per (row block, part, communication warp)
          __threadfence_system();
          const size_t word = (static_cast<size_t>(c.rank * chunks + ch) * parts + part) * COMM_WARPS + (cw >> 5);
          if (mm) {
            multimem_red_release_max(reinterpret_cast<uint32_t*>(c.mc_base + c.flag_off) + word, c.epoch);
          } else {
            for (int w = 0; w < c.world; ++w)
              st_release_sys(reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(c.peer_bufs[w]) + c.flag_off) + word, c.epoch);
          }
        }
      }
    } else {
      const int rows_per_rank = p.M / c.world;
      // This CTA reduces, of the tiles it PRODUCES itself (same raster walk as its MMA warp), the ones this rank owns.
      // Every rank launches the same grid, so a tile is produced by the CTA of the same index on every rank: a CTA
      // only ever waits for its namesakes on the peers. If some CTAs of the grid are not resident yet (their SMs are
      // held by another kernel - a point-to-point transfer that is itself waiting for its peer), the resident ones
      // still finish and leave, which is what lets the late ones in; nothing here needs the whole grid at once.
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        coords(t, tm, tn);
        const int tile = tm * p.tiles_n + tn;
        if (tile_owner(c, tile, tm, p.tiles_m) != c.rank) continue;
        const uint64_t tw0 = trace ? globaltimer_ns() : 0;
        ok = warp_wait_words(my_flags + static_cast<size_t>(tile) * c.world * 4, c.world * 4, c.epoch, abort_flag, p.err);
        if (!ok) break;
        const uint64_t tw1 = trace ? globaltimer_ns() : 0;
        if (trace && cw == 0) trace[6] += tw1 - tw0;
        const int m0 = tm * BM, n0 = tn * BN;
        const int rows = min(BM, p.M - m0), cols = min(BN, p.N - n0);
        const int vpr = cols / 8;
        const int total = rows * vpr;
        constexpr int UNR = 8;  // 16-byte requests in flight per thread: NVLink round trips are ~10 us under load
        for (int base = cw; base < ((c.debug & 2) ? 0 : total); base += COMM_THREADS * UNR) {
          uint4 v[UNR];
          size_t off[UNR];
#pragma unroll
          for (int j = 0; j < UNR; ++j) {
            const int idx = base + j * COMM_THREADS;
            if (idx < total) {
              const int r = idx / vpr, q = idx % vpr;
              off[j] = c.data_off + (static_cast<size_t>(m0 + r) * p.N + n0 + q * 8) * 2;
              if (mm) v[j] = mm_ld_reduce_16(c.mc_base + off[j], fp16);
            }
          }
          if (!mm) {
            // plain peer loads: fetch every rank's copy of a vector before adding them up
#pragma unroll
            for (int j = 0; j < UNR; ++j) {
              const int idx = base + j * COMM_THREADS;
              if (idx < total) {
                uint4 part[8];  // the launcher refuses peer mode beyond 8 ranks
#pragma unroll
                for (int w = 0; w < 8; ++w)
                  if (w < c.world)
                    part[w] = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(c.peer_bufs[w]) + off[j]);
                float acc[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                  if (w < c.world) {
                    float t[8];
                    unpack8(part[w], t, fp16);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] += t[e];
                  }
                }
                v[j].x = pack2(acc[0], acc[1], fp16); v[j].y = pack2(acc[2], acc[3], fp16);
                v[j].z = pack2(acc[4], acc[5], fp16); v[j].w = pack2(acc[6], acc[7], fp16);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < UNR; ++j) {
            const int idx = base + j * COMM_THREADS;
            if (idx < total) {
              if (c.mode == COMM_ALLREDUCE) {
                if (mm) {
                  mm_st_16(c.mc_base + off[j], v[j]);
                } else {
                  for (int w = 0; w < c.world; ++w)
                    *reinterpret_cast<uint4*>(static_cast<uint8_t*>(c.peer_bufs[w]) + off[j]) = v[j];
                }
              } else {
                const int r = idx / vpr, q = idx % vpr;
                uint16_t* o = reinterpret_cast<uint16_t*>(c.out) +
                              static_cast<size_t>(m0 + r - c.rank * rows_per_rank) * c.ld_out + n0 + q * 8;
                *reinterpret_cast<uint4*>(o) = v[j];
              }
            }
          }
        }
        if (trace && cw == 0) trace[7] += globaltimer_ns() - tw1;
        if (c.mode == COMM_ALLREDUCE) {
          // tell every rank that one more tile of the result is final
          __syncwarp();
          if ((cw & 31) == 0) {
            __threadfence_system();
            if (mm) {
              multimem_red_release_add(reinterpret_cast<uint32_t*>(c.mc_base + c.done_off), 1u);
            } else {
              for (int w = 0; w < c.world; ++w)
                red_release_sys_add(reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(c.peer_bufs[w]) + c.done_off), 1u);
            }
          }
        }
      }
      if (c.mode == COMM_ALLREDUCE && ok && cw == 0 && blockIdx.x == gridDim.x - 1) {
        // the result is complete on this rank once every tile of every owner has been broadcast. ONE CTA waits for
        // that (the kernel cannot end before its last CTA does); the others leave as soon as their own tiles are done.
        // It is the CTA with the highest index: blocks are handed to the SMs in index order, so by the time it
        // runs every other CTA has been started and none is left waiting for the slot it holds
        wait_flag_ge(reinterpret_cast<const uint32_t*>(my_base + c.done_off), c.done_target, abort_flag, p.err);
      }
      if (trace && cw == 0) trace[4] = globaltimer_ns();
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

}  // namespace oslo
