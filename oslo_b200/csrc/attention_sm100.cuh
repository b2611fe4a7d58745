// Pieces shared by the tcgen05 flash-attention kernels (forward: attention_sm100.cu, backward:
// attention_bwd_sm100.cu): 4-D TMA loads addressed by (d, seq, head, batch), TMEM stores, 16-bit packing, and
// the host-side tensor-map builder for [B, H, S, D] views with arbitrary (16-byte aligned) strides.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include <algorithm>
#include <cstdlib>

#include "oslo_kernels.h"
#include "ptx.cuh"

namespace oslo {

int make_tma_nd_16bit(CUtensorMap* map, const void* ptr, int rank, const uint64_t* dims, const uint64_t* strides_elems,
                      const uint32_t* box, bool fp16);

constexpr int FA_BM = 128;
constexpr int FA_THREADS = 192;
constexpr float FA_LOG2E = 1.4426950408889634f;
constexpr float FA_LN2 = 0.6931471805599453f;
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// load a [rows x 64] box whose rows run along the sequence dim; pos[] says where (seq, head, batch) go
__device__ __forceinline__ void tma_load_rows(uint32_t dst, const CUtensorMap* map, uint32_t bar, int d0, int s0, int h,
                                              int b, const int* pos) {
  auto pick = [&](int slot) { return pos[0] == slot ? s0 : (pos[1] == slot ? h : b); };
  tma_load_4d(dst, map, bar, d0, pick(0), pick(1), pick(2));
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t fa_pack2(float a, float b, bool fp16) {
  if (fp16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// 4-D map {D, x, y, z} over a [B, H, S, D] view given by element strides; the three outer dims are ordered by
// ascending stride and `pos` records where (seq, head, batch) ended up. The box is {64, rows} along D and seq.
static inline int make_qkv_map(CUtensorMap* map, const void* ptr, int B, int H, int S, int D, long long sb, long long sh,
                        long long ss, int rows, bool fp16, int* pos) {
  struct Dim { long long stride; uint64_t size; int kind; };
  Dim dd[3] = {{ss, static_cast<uint64_t>(S), 0}, {sh, static_cast<uint64_t>(H), 1}, {sb, static_cast<uint64_t>(B), 2}};
  std::stable_sort(dd, dd + 3, [](const Dim& a, const Dim& b) { return a.stride < b.stride; });
  uint64_t dims[4] = {static_cast<uint64_t>(D), 0, 0, 0};
  uint64_t strides[3];
  uint32_t box[4] = {64, 1, 1, 1};
  for (int i = 0; i < 3; ++i) {
    if (dd[i].stride <= 0) return -102;
    dims[1 + i] = dd[i].size;
    strides[i] = static_cast<uint64_t>(dd[i].stride);
    pos[dd[i].kind] = i;
    if (dd[i].kind == 0) box[1 + i] = static_cast<uint32_t>(rows);
  }
  return make_tma_nd_16bit(map, ptr, 4, dims, strides, box, fp16);
}

}  // namespace oslo
