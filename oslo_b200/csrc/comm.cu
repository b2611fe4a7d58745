// Collectives over symmetric memory (every rank holds the same buffer at peer-mapped addresses, plus an
// NVSwitch multicast mapping of it). Cross-GPU synchronisation uses per-(block, peer) signal words with a
// compare-and-swap handshake; every spin is bounded and reports through the error word.
//
//  * multimem mode (NVLS): rank r owns slice r of the buffer; it issues multimem.ld_reduce on the multicast
//    address (the switch returns the sum over all ranks) and multimem.st to broadcast the reduced slice back
//    into every rank's buffer - each byte crosses this GPU's links once in each direction.
//  * peer mode: each rank reads every peer's buffer directly (one-shot) and writes the sum to `out`.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "oslo_kernels.h"
#include "ptx.cuh"

namespace oslo {

__device__ __forceinline__ bool signal_put(uint32_t* addr, int* err) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    uint32_t old;
    asm volatile("atom.global.release.sys.cas.b32 %0, [%1], 0, 1;" : "=r"(old) : "l"(addr) : "memory");
    if (old == 0) return true;
    if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > OSLO_WAIT_LIMIT_NS) {
      if (err) atomicCAS(err, 0, ERR_WAIT_PEER);
      return false;
    }
  }
}
__device__ __forceinline__ bool signal_wait(uint32_t* addr, int* err) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    uint32_t old;
    asm volatile("atom.global.acquire.sys.cas.b32 %0, [%1], 1, 0;" : "=r"(old) : "l"(addr) : "memory");
    if (old == 1) return true;
    if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > OSLO_WAIT_LIMIT_NS) {
      if (err) atomicCAS(err, 0, ERR_WAIT_PEER);
      return false;
    }
  }
}

// all ranks' blocks with the same blockIdx meet; slot layout: [block][source rank]
__device__ __forceinline__ bool block_barrier_all_ranks(uint32_t* const* signal_ptrs, int rank, int world, int slot0,
                                                        int* err) {
  __shared__ int ok_s;
  __syncthreads();
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < world) {
    __threadfence_system();
    const int peer = threadIdx.x;
    bool ok = signal_put(signal_ptrs[peer] + slot0 + blockIdx.x * world + rank, err);
    ok = ok && signal_wait(signal_ptrs[rank] + slot0 + blockIdx.x * world + peer, err);
    if (!ok) ok_s = 0;
  }
  __syncthreads();
  return ok_s != 0;
}

template <bool FP16>
__device__ __forceinline__ uint4 multimem_ld_reduce(const void* mc_addr) {
  uint4 v;
  if (FP16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}

template <bool FP16>
__device__ __forceinline__ uint4 add8(const uint4& a, const uint4& b) {
  uint4 r;
  const uint32_t* pa = &a.x; const uint32_t* pb = &b.x; uint32_t* pr = &r.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (FP16) {
      const float2 x = __half22float2(*reinterpret_cast<const __half2*>(pa + i));
      const float2 y = __half22float2(*reinterpret_cast<const __half2*>(pb + i));
      __half2 h = __floats2half2_rn(x.x + y.x, x.y + y.y);
      pr[i] = *reinterpret_cast<uint32_t*>(&h);
    } else {
      const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pa + i));
      const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pb + i));
      __nv_bfloat162 h = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
      pr[i] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  return r;
}

// n16 = number of 16-byte vectors in the buffer
template <bool FP16>
__global__ void __launch_bounds__(512) allreduce_symm_kernel(void* const* peer_ptrs, void* mc_ptr,
                                                             uint32_t* const* signal_ptrs, void* out, long long n16,
                                                             int rank, int world, int use_multimem, int* err) {
  if (!block_barrier_all_ranks(signal_ptrs, rank, world, 0, err)) return;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  if (use_multimem) {
    const long long per = (n16 + world - 1) / world;
    const long long lo = per * rank, hi = min(n16, lo + per);
    uint4* mc = reinterpret_cast<uint4*>(mc_ptr);
    for (long long i = lo + tid; i < hi; i += nthreads) {
      const uint4 v = multimem_ld_reduce<FP16>(mc + i);
      multimem_st(mc + i, v);
    }
    if (!block_barrier_all_ranks(signal_ptrs, rank, world, gridDim.x * world, err)) return;
    if (out != peer_ptrs[rank]) {
      const uint4* src = reinterpret_cast<const uint4*>(peer_ptrs[rank]);
      uint4* dst = reinterpret_cast<uint4*>(out);
      for (long long i = tid; i < n16; i += nthreads) dst[i] = src[i];
      // the staging region is shared with other collectives of this workspace: nobody may write into it again
      // (a peer's next call) before every rank has copied its result out. The first barrier's signal words are
      // free again by now (each was consumed before its owner could reach the second barrier).
      block_barrier_all_ranks(signal_ptrs, rank, world, 0, err);
    }
  } else {
    uint4* dst = reinterpret_cast<uint4*>(out);
    for (long long i = tid; i < n16; i += nthreads) {
      uint4 acc = reinterpret_cast<const uint4*>(peer_ptrs[rank])[i];
      for (int r = 1; r < world; ++r) {
        const int peer = (rank + r) % world;
        acc = add8<FP16>(acc, reinterpret_cast<const uint4*>(peer_ptrs[peer])[i]);
      }
      dst[i] = acc;
    }
    // peers must not overwrite their buffers while others still read them
    block_barrier_all_ranks(signal_ptrs, rank, world, gridDim.x * world, err);
  }
}

// One-shot all-reduce for latency-bound sizes, one kernel and one cross-rank barrier per call:
//   1. every block copies its slice of `in` into this rank's symmetric staging buffer (half `parity`),
//   2. meets the same block of every other rank,
//   3. sums the slice over all ranks (multimem.ld_reduce, or peer loads) straight into `out` (may alias `in`).
// The two staging halves alternate per call; the parity lives in device memory (one counter per block, bumped by
// the block itself), so a replayed CUDA graph keeps alternating. A half is only rewritten two calls later, and a
// rank can get there only after every rank has passed the barrier of the call in between, i.e. has finished
// reading: no trailing barrier is needed.
template <bool FP16>
__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const void* in, void* out, void* const* peer_ptrs,
                                                                void* mc_ptr, uint32_t* const* signal_ptrs,
                                                                uint32_t* counters, long long n16, long long stage_off16,
                                                                long long half16, int rank, int world, int use_multimem,
                                                                int* err) {
  const uint32_t parity = counters[blockIdx.x] & 1u;
  const long long base = stage_off16 + parity * half16;
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  uint4* mine = reinterpret_cast<uint4*>(peer_ptrs[rank]) + base;
  for (long long i = tid; i < n16; i += nthreads) mine[i] = reinterpret_cast<const uint4*>(in)[i];
  if (!block_barrier_all_ranks(signal_ptrs, rank, world, 0, err)) return;
  uint4* dst = reinterpret_cast<uint4*>(out);
  if (use_multimem) {
    const uint4* mc = reinterpret_cast<const uint4*>(mc_ptr) + base;
    for (long long i = tid; i < n16; i += nthreads) dst[i] = multimem_ld_reduce<FP16>(mc + i);
  } else {
    for (long long i = tid; i < n16; i += nthreads) {
      uint4 acc = mine[i];
      for (int r = 1; r < world; ++r) {
        const int peer = (rank + r) % world;
        acc = add8<FP16>(acc, (reinterpret_cast<const uint4*>(peer_ptrs[peer]) + base)[i]);
      }
      dst[i] = acc;
    }
  }
  if (threadIdx.x == 0) counters[blockIdx.x] += 1;
}

// Bounded wait on a word of ordinary device memory, with a caller-chosen limit: the same loop shape as the waits on
// peer flags (acquire load, timer check, error word, clean return). It exists so that the give-up path can be
// exercised by a test with a flag that nothing sets and a limit of a fraction of a second.
__global__ void wait_probe_kernel(const uint32_t* flag, uint32_t target, unsigned long long limit_ns, int* err,
                                  unsigned long long* waited_ns) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t v;
  while (true) {
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - target) >= 0) break;
    if (globaltimer_ns() - t0 > limit_ns) {
      if (err) atomicCAS(err, 0, ERR_WAIT_PEER);
      break;
    }
    __nanosleep(200);
  }
  if (waited_ns) *waited_ns = globaltimer_ns() - t0;
}

// Vocab-parallel embedding lookup fused with its collective. Exactly one rank owns the row of a token id, so no
// reduction is needed: the owner stores the row into EVERY rank's staging buffer (multimem.st through the switch,
// or one plain store per peer), block b of every rank handles the same token range, meets block b of the other
// ranks once, and copies its range out of its own staging buffer. Half as many bytes cross the links as in the
// "masked lookup + all-reduce" form, and the lookup, mask, zero-fill and collective are one launch. Staging halves
// alternate by a device-side per-block counter; the launcher always starts the same number of blocks so that all
// counters stay equal (the token -> block split changes with the token count, unlike the one-shot all-reduce's fixed
// 512 vectors per block). Reuse of a half two calls later is then safe without a trailing barrier: a rank that writes
// in call n+2 has finished call n+1, whose barriers every peer block reached only after the peer's call n kernel -
// all of its copy-outs - had completed (launches of one stream do not overlap).
template <typename T>
__global__ void __launch_bounds__(512) vocab_embed_kernel(const long long* __restrict__ ids, const T* __restrict__ weight,
                                                          T* __restrict__ out, void* const* peer_ptrs, void* mc_ptr,
                                                          uint32_t* const* signal_ptrs, uint32_t* counters,
                                                          long long tokens, int H, long long lo, long long hi,
                                                          long long half16, int rank, int world, int use_multimem,
                                                          int* err) {
  const uint32_t parity = counters[blockIdx.x] & 1u;
  const long long base16 = parity * half16;
  const int vpr = H / 8;                                         // 16-byte vectors per row
  const long long per = (tokens + gridDim.x - 1) / gridDim.x;    // tokens of this block (same split on every rank)
  const long long t0 = blockIdx.x * per, t1 = min(tokens, t0 + per);
  const long long total = (t1 > t0 ? t1 - t0 : 0) * vpr;
  for (long long i = threadIdx.x; i < total; i += blockDim.x) {
    const long long t = t0 + i / vpr;
    const int v = static_cast<int>(i % vpr);
    const long long id = ids[t];
    if (id >= lo && id < hi) {
      const uint4 val = reinterpret_cast<const uint4*>(weight + (id - lo) * H)[v];
      const long long off = base16 + t * vpr + v;
      if (use_multimem) {
        multimem_st(reinterpret_cast<uint4*>(mc_ptr) + off, val);
      } else {
        for (int r = 0; r < world; ++r) (reinterpret_cast<uint4*>(peer_ptrs[r]) + off)[0] = val;
      }
    }
  }
  if (!block_barrier_all_ranks(signal_ptrs, rank, world, 0, err)) return;
  const uint4* mine = reinterpret_cast<const uint4*>(peer_ptrs[rank]) + base16 + t0 * vpr;
  uint4* dst = reinterpret_cast<uint4*>(out) + t0 * vpr;
  for (long long i = threadIdx.x; i < total; i += blockDim.x) dst[i] = mine[i];
  if (threadIdx.x == 0) counters[blockIdx.x] += 1;
}

// ---------------------------------------------------------------------------------------------------------------
// Data-parallel gradient reduce-scatter and parameter all-gather, in place on SYMMETRIC flat buffers (ZeRO-1).
//
// The flat gradient buffer and the flat parameter buffer of a data-parallel replica live in symmetric memory (same
// layout on every rank, peer-mapped, plus the NVSwitch multicast mapping). Rank r owns vectors
// [r * shard16, (r + 1) * shard16) of either buffer. Both kernels work on one bucket [lo16, hi16) of the buffer:
//
//   reduce-scatter: all ranks meet (everybody's bucket is complete), then every rank pulls the SUM of the part of the
//     bucket that lies in ITS shard - multimem.ld_reduce (the switch adds the ranks' copies, fp32 accumulation) or
//     plain peer loads added in fp32 - and stores it into its own gradient buffer. Half the bytes of an all-reduce:
//     nothing is broadcast back, because only the owner updates those parameters. A trailing meeting keeps every
//     rank from touching the bucket again (zeroing it for the next step) while an owner still reads it.
//   all-gather: all ranks meet (nobody still reads the old parameters), every rank stores the part of the bucket that
//     lies in its shard - the parameters its optimizer step just wrote - into every rank's buffer (multimem.st, or
//     one plain store per peer), and a second meeting makes the kernel's completion mean "every rank's part of this
//     bucket has landed here".
//
// Every rank launches the same grid for a bucket (it depends on the bucket's size only).
template <bool FP16>
__device__ __forceinline__ void accumulate8(float (&acc)[8], const uint4& v) {
  const uint32_t* pv = &v.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t;
    if (FP16) t = __half22float2(*reinterpret_cast<const __half2*>(pv + i));
    else t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(pv + i));
    acc[2 * i] += t.x;
    acc[2 * i + 1] += t.y;
  }
}
template <bool FP16>
__device__ __forceinline__ uint4 pack8(const float (&acc)[8]) {
  uint4 r;
  uint32_t* pr = &r.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (FP16) {
      __half2 h = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
      pr[i] = *reinterpret_cast<uint32_t*>(&h);
    } else {
      __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      pr[i] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  return r;
}

constexpr int DP_UNROLL = 8;   // 16-byte requests in flight per thread

template <bool FP16>
__global__ void __launch_bounds__(512) dp_reduce_scatter_kernel(void* const* peer_ptrs, void* mc_ptr,
                                                                uint32_t* const* signal_ptrs, long long lo16,
                                                                long long hi16, long long shard16, int rank, int world,
                                                                int use_multimem, int* err) {
  if (!block_barrier_all_ranks(signal_ptrs, rank, world, 0, err)) return;
  const long long a = max(lo16, shard16 * rank), b = min(hi16, shard16 * (rank + 1));
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  uint4* own = reinterpret_cast<uint4*>(peer_ptrs[rank]);
  if (use_multimem) {
    const uint4* mc = reinterpret_cast<const uint4*>(mc_ptr);
    for (long long i0 = a + tid; i0 < b; i0 += nthreads * DP_UNROLL) {
      uint4 v[DP_UNROLL];
#pragma unroll
      for (int j = 0; j < DP_UNROLL; ++j) {
        const long long i = i0 + j * nthreads;
        if (i < b) v[j] = multimem_ld_reduce<FP16>(mc + i);
      }
#pragma unroll
      for (int j = 0; j < DP_UNROLL; ++j) {
        const long long i = i0 + j * nthreads;
        if (i < b) own[i] = v[j];
      }
    }
  } else {
    for (long long i = a + tid; i < b; i += nthreads) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int r = 0; r < world; ++r) {
        const int peer = (rank + r) % world;
        accumulate8<FP16>(acc, reinterpret_cast<const uint4*>(peer_ptrs[peer])[i]);
      }
      own[i] = pack8<FP16>(acc);
    }
  }
  block_barrier_all_ranks(signal_ptrs, rank, world, gridDim.x * world, err);
}

__global__ void __launch_bounds__(512) dp_all_gather_kernel(void* const* peer_ptrs, void* mc_ptr,
                                                            uint32_t* const* signal_ptrs, long long lo16, long long hi16,
                                                            long long shard16, int rank, int world, int use_multimem,
                                                            int* err) {
  if (!block_barrier_all_ranks(signal_ptrs, rank, world, 0, err)) return;
  const long long a = max(lo16, shard16 * rank), b = min(hi16, shard16 * (rank + 1));
  const long long tid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
  const uint4* own = reinterpret_cast<const uint4*>(peer_ptrs[rank]);
  for (long long i0 = a + tid; i0 < b; i0 += nthreads * DP_UNROLL) {
    uint4 v[DP_UNROLL];
#pragma unroll
    for (int j = 0; j < DP_UNROLL; ++j) {
      const long long i = i0 + j * nthreads;
      if (i < b) v[j] = own[i];
    }
#pragma unroll
    for (int j = 0; j < DP_UNROLL; ++j) {
      const long long i = i0 + j * nthreads;
      if (i < b) {
        if (use_multimem) {
          multimem_st(reinterpret_cast<uint4*>(mc_ptr) + i, v[j]);
        } else {
          for (int r = 1; r < world; ++r) reinterpret_cast<uint4*>(peer_ptrs[(rank + r) % world])[i] = v[j];
        }
      }
    }
  }
  block_barrier_all_ranks(signal_ptrs, rank, world, gridDim.x * world, err);
}

// Vocabulary-parallel cross-entropy: every rank holds (max, sum exp(x - max), label logit) of its vocabulary shard for
// n rows; all ranks need the combination over the shards. One kernel, one meeting: copy the three vectors into this
// rank's staging half in symmetric memory, meet, read every rank's triple with plain peer loads and combine in a
// fixed rank order (so every rank computes bit-identical results): gm = max_r m_r, s = sum_r s_r exp(m_r - gm),
// t = sum_r t_r. `cap` floats per vector per half; the launcher always starts the same grid, so the per-block
// half parities stay equal and a half is rewritten only after every rank has finished the call in between.
__global__ void __launch_bounds__(256) ce_combine_kernel(const float* __restrict__ mx, const float* __restrict__ se,
                                                         const float* __restrict__ tg, float* __restrict__ out_mx,
                                                         float* __restrict__ out_se, float* __restrict__ out_tg,
                                                         void* const* peer_ptrs, uint32_t* const* signal_ptrs,
                                                         uint32_t* counters, int n, int cap, int rank, int world,
                                                         int* err) {
  const uint32_t parity = counters[blockIdx.x] & 1u;
  const size_t base = static_cast<size_t>(parity) * 3 * cap;
  float* mine = reinterpret_cast<float*>(peer_ptrs[rank]) + base;
  const int tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
  for (int i = tid; i < n; i += nthreads) {
    mine[i] = mx[i];
    mine[cap + i] = se[i];
    mine[2 * cap + i] = tg[i];
  }
  if (!block_barrier_all_ranks(signal_ptrs, rank, world, 0, err)) return;
  for (int i = tid; i < n; i += nthreads) {
    float gm = -3.0e38f;
    for (int r = 0; r < world; ++r) gm = fmaxf(gm, (reinterpret_cast<const float*>(peer_ptrs[r]) + base)[i]);
    float s = 0.f, t = 0.f;
    for (int r = 0; r < world; ++r) {
      const float* pr = reinterpret_cast<const float*>(peer_ptrs[r]) + base;
      s += pr[cap + i] * __expf(pr[i] - gm);
      t += pr[2 * cap + i];
    }
    out_mx[i] = gm;
    out_se[i] = s;
    out_tg[i] = t;
  }
  if (threadIdx.x == 0) counters[blockIdx.x] += 1;
}

}  // namespace oslo

// mx / se / tg and the outputs: fp32 [n] (outputs may alias the inputs). The symmetric buffer holds 2 x 3 x cap floats;
// counters: device uint32[>= 8], zeroed once.
extern "C" int oslo_ce_combine(const float* mx, const float* se, const float* tg, float* out_mx, float* out_se,
                               float* out_tg, void* const* peer_ptrs_dev, uint32_t* const* signal_ptrs_dev,
                               uint32_t* counters, int n, int cap, int rank, int world, int* err_word,
                               cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n > cap || world > 16 || rank < 0 || rank >= world) return -3;
  oslo::ce_combine_kernel<<<8, 256, 0, stream>>>(mx, se, tg, out_mx, out_se, out_tg, peer_ptrs_dev, signal_ptrs_dev,
                                                 counters, n, cap, rank, world, err_word);
  return static_cast<int>(cudaGetLastError());
}

// Bucket [lo, hi) (element indices, multiples of 8) of a symmetric flat buffer of 16-bit elements whose rank r owns
// elements [r * shard, (r + 1) * shard). reduce_scatter: every rank's own part of the bucket becomes the sum over all
// ranks (in place, in its own buffer); all_gather: every rank's own part is copied into all ranks' buffers.
static int dp_grid(long long n16, int world) {
  int max_blocks = 2048 / 4 / (2 * world);   // two meetings x blocks x world signal words within the 2 KiB signal pad
  if (max_blocks > 64) max_blocks = 64;
  long long want = (n16 + 512LL * oslo::DP_UNROLL - 1) / (512LL * oslo::DP_UNROLL);
  return static_cast<int>(want < 1 ? 1 : (want > max_blocks ? max_blocks : want));
}
extern "C" int oslo_dp_reduce_scatter(void* const* peer_ptrs_dev, void* mc_ptr, uint32_t* const* signal_ptrs_dev,
                                      long long lo, long long hi, long long shard, int rank, int world, int dtype,
                                      int use_multimem, int* err_word, cudaStream_t stream) {
  using namespace oslo;
  if (hi <= lo) return 0;
  if (lo % 8 || hi % 8 || shard % 8 || lo < 0 || shard <= 0 || rank < 0 || rank >= world) return -3;
  if (world > 16) return -4;
  const int blocks = dp_grid((hi - lo) / 8, world);
  const int mm = (use_multimem && mc_ptr != nullptr) ? 1 : 0;
  if (dtype == OSLO_DT_FP16)
    dp_reduce_scatter_kernel<true><<<blocks, 512, 0, stream>>>(peer_ptrs_dev, mc_ptr, signal_ptrs_dev, lo / 8, hi / 8,
                                                               shard / 8, rank, world, mm, err_word);
  else if (dtype == OSLO_DT_BF16)
    dp_reduce_scatter_kernel<false><<<blocks, 512, 0, stream>>>(peer_ptrs_dev, mc_ptr, signal_ptrs_dev, lo / 8, hi / 8,
                                                                shard / 8, rank, world, mm, err_word);
  else
    return -2;
  return static_cast<int>(cudaGetLastError());
}
extern "C" int oslo_dp_all_gather(void* const* peer_ptrs_dev, void* mc_ptr, uint32_t* const* signal_ptrs_dev,
                                  long long lo, long long hi, long long shard, int rank, int world, int use_multimem,
                                  int* err_word, cudaStream_t stream) {
  using namespace oslo;
  if (hi <= lo) return 0;
  if (lo % 8 || hi % 8 || shard % 8 || lo < 0 || shard <= 0 || rank < 0 || rank >= world) return -3;
  if (world > 16) return -4;
  const int blocks = dp_grid((hi - lo) / 8, world);
  const int mm = (use_multimem && mc_ptr != nullptr) ? 1 : 0;
  dp_all_gather_kernel<<<blocks, 512, 0, stream>>>(peer_ptrs_dev, mc_ptr, signal_ptrs_dev, lo / 8, hi / 8, shard / 8, rank,
                                                   world, mm, err_word);
  return static_cast<int>(cudaGetLastError());
}

// one thread waits until *flag >= target or limit_ns (capped at 1 s) has passed; on expiry the error word gets
// ERR_WAIT_PEER. waited_ns (device, optional) receives the time spent.
extern "C" int oslo_wait_probe(const uint32_t* flag, uint32_t target, unsigned long long limit_ns, int* err_word,
                               unsigned long long* waited_ns, cudaStream_t stream) {
  if (limit_ns > 1000000000ull) limit_ns = 1000000000ull;
  oslo::wait_probe_kernel<<<1, 1, 0, stream>>>(flag, target, limit_ns, err_word, waited_ns);
  return static_cast<int>(cudaGetLastError());
}

// out [tokens, H] = rows of the vocabulary-sharded weight [hi - lo, H] (this rank owns ids in [lo, hi)); every id must
// be owned by exactly one rank of the group. `half_bytes`: size of one of the two staging halves at the start of
// the symmetric buffer (tokens * H * 2 <= half_bytes). `counters`: device uint32[>= 64], zeroed once.
extern "C" int oslo_vocab_embed(const long long* ids, const void* weight, void* out, void* const* peer_ptrs_dev,
                                void* mc_ptr, uint32_t* const* signal_ptrs_dev, uint32_t* counters, long long tokens,
                                int H, long long lo, long long hi, long long half_bytes, int rank, int world, int dtype,
                                int use_multimem, int* err_word, int num_sms, cudaStream_t stream) {
  using namespace oslo;
  if (tokens <= 0) return 0;
  if (H % 8 || half_bytes % 16 || tokens * H * 2 > half_bytes || world > 16) return -3;
  int max_blocks = 2048 / 4 / (2 * world);
  if (max_blocks > 64) max_blocks = 64;
  if (max_blocks > num_sms) max_blocks = num_sms;
  // Always the same grid, whatever the token count: blocks without tokens still meet their peers and bump their
  // counter, so every block's parity moves in lockstep and "the other half" means the same thing for every token
  // offset on every rank. (With a grid that followed the token count, a short call - a decode step - would advance
  // only the first counters, and two later calls could then put one token offset into the same half twice in a row.)
  const int blocks = max_blocks;
  if (dtype == OSLO_DT_BF16)
    vocab_embed_kernel<__nv_bfloat16><<<blocks, 512, 0, stream>>>(ids, (const __nv_bfloat16*)weight, (__nv_bfloat16*)out,
                                                                  peer_ptrs_dev, mc_ptr, signal_ptrs_dev, counters, tokens,
                                                                  H, lo, hi, half_bytes / 16, rank, world, use_multimem,
                                                                  err_word);
  else if (dtype == OSLO_DT_FP16)
    vocab_embed_kernel<__half><<<blocks, 512, 0, stream>>>(ids, (const __half*)weight, (__half*)out, peer_ptrs_dev, mc_ptr,
                                                           signal_ptrs_dev, counters, tokens, H, lo, hi, half_bytes / 16,
                                                           rank, world, use_multimem, err_word);
  else
    return -2;
  return static_cast<int>(cudaGetLastError());
}

// `counters`: device uint32[>= 64], zero-initialised once, owned by this rank. `stage_off` / `half_bytes`: byte
// offset of the two staging halves inside the symmetric buffer and the size of one half (n * 2 <= half_bytes).
extern "C" int oslo_allreduce_oneshot(const void* in, void* out, void* const* peer_ptrs_dev, void* mc_ptr,
                                      uint32_t* const* signal_ptrs_dev, uint32_t* counters, long long n,
                                      long long stage_off, long long half_bytes, int rank, int world, int dtype,
                                      int use_multimem, int* err_word, cudaStream_t stream) {
  using namespace oslo;
  if (n == 0) return 0;
  if (n % 8 || stage_off % 16 || half_bytes % 16 || n * 2 > half_bytes) return -3;
  if (world > 16) return -4;
  const long long n16 = n / 8;
  int max_blocks = 2048 / 4 / (2 * world);   // same signal-pad budget as the two-shot kernel
  if (max_blocks > 64) max_blocks = 64;
  long long want = (n16 + 511) / 512;
  const int blocks = static_cast<int>(want < 1 ? 1 : (want > max_blocks ? max_blocks : want));
  if (dtype == OSLO_DT_FP16)
    allreduce_oneshot_kernel<true><<<blocks, 512, 0, stream>>>(in, out, peer_ptrs_dev, mc_ptr, signal_ptrs_dev, counters,
                                                               n16, stage_off / 16, half_bytes / 16, rank, world,
                                                               use_multimem, err_word);
  else if (dtype == OSLO_DT_BF16)
    allreduce_oneshot_kernel<false><<<blocks, 512, 0, stream>>>(in, out, peer_ptrs_dev, mc_ptr, signal_ptrs_dev, counters,
                                                                n16, stage_off / 16, half_bytes / 16, rank, world,
                                                                use_multimem, err_word);
  else
    return -2;
  return static_cast<int>(cudaGetLastError());
}

extern "C" int oslo_allreduce_symm(void* const* peer_ptrs_dev, void* mc_ptr, uint32_t* const* signal_ptrs_dev,
                                   void* out, long long n, int rank, int world, int dtype, int use_multimem,
                                   int* err_word, cudaStream_t stream) {
  using namespace oslo;
  if (n == 0) return 0;
  if (n % 8) return -3;  // 16-byte vectors of 16-bit elements
  if (world > 16) return -4;
  const long long n16 = n / 8;
  // the signal pad holds 2 barriers x blocks x world 32-bit slots; keep it within 2 KiB
  int max_blocks = 2048 / 4 / (2 * world);
  long long want = (n16 / (use_multimem ? world : 1) + 511) / 512;
  int blocks = static_cast<int>(want < 1 ? 1 : (want > max_blocks ? max_blocks : want));
  if (dtype == OSLO_DT_FP16)
    allreduce_symm_kernel<true><<<blocks, 512, 0, stream>>>(peer_ptrs_dev, mc_ptr, signal_ptrs_dev, out, n16, rank,
                                                            world, use_multimem, err_word);
  else if (dtype == OSLO_DT_BF16)
    allreduce_symm_kernel<false><<<blocks, 512, 0, stream>>>(peer_ptrs_dev, mc_ptr, signal_ptrs_dev, out, n16, rank,
                                                             world, use_multimem, err_word);
  else
    return -2;
  return static_cast<int>(cudaGetLastError());
}
