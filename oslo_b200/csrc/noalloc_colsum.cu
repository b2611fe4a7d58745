// Allocation-free column sums: see oslo_noalloc.h for who needs this and the rules of use.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "oslo_kernels.h"
#include "oslo_noalloc.h"

namespace {

// The workspace. In host code this name is only a handle for cudaGetSymbolAddress - it is NOT a device
// address and must never be passed to a kernel directly.
static __device__ __align__(256) float g_colsum_scratch[OSLO_NOALLOC_COLSUM_PARTS * OSLO_NOALLOC_COLSUM_MAX_COLS];

template <typename T> __device__ __forceinline__ float as_float(T v);
template <> __device__ __forceinline__ float as_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float as_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float as_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// grid (column blocks, parts): thread = one column, strides over the rows of its part; writes part[p, c]
template <typename T>
__global__ void colsum_part_kernel(const T* __restrict__ x, float* __restrict__ part, int rows, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int r = blockIdx.y; r < rows; r += gridDim.y) s += as_float(x[static_cast<size_t>(r) * cols + c]);
  part[static_cast<size_t>(blockIdx.y) * cols + c] = s;
}
__global__ void colsum_final_kernel(const float* __restrict__ part, float* __restrict__ out, int parts, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += part[static_cast<size_t>(p) * cols + c];
  out[c] = s;
}

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

// Device address of the workspace on the current device, resolved once per device.
int scratch_for_current_device(float** addr) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kMaxDevices) return -3;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_colsum_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (p == nullptr) return -3;
    g_scratch_addr[dev] = p;
  }
  *addr = g_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int oslo_colsum_noalloc(const void* x, float* out, int rows, int cols, int dtype, cudaStream_t stream) {
  if (rows < 0 || cols < 0 || (rows > 0 && cols > 0 && (x == nullptr || out == nullptr))) return -3;
  if (cols > OSLO_NOALLOC_COLSUM_MAX_COLS) return -10;  // the built-in workspace is too small: nothing launched
  if (dtype != OSLO_DT_BF16 && dtype != OSLO_DT_FP16 && dtype != OSLO_DT_FP32) return -2;
  if (cols == 0) return 0;
  {
    // an error left behind by an earlier launch of somebody else is reported as such, before this call's launches
    const cudaError_t stale = cudaGetLastError();
    if (stale != cudaSuccess) return static_cast<int>(stale);
  }
  float* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  int parts = rows < OSLO_NOALLOC_COLSUM_PARTS ? rows : OSLO_NOALLOC_COLSUM_PARTS;
  if (parts < 1) parts = 1;  // rows == 0: one part of zeros, so out becomes all zero
  const dim3 grid((cols + 127) / 128, parts);
  if (dtype == OSLO_DT_BF16)
    colsum_part_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), scratch, rows, cols);
  else if (dtype == OSLO_DT_FP16)
    colsum_part_kernel<__half><<<grid, 128, 0, stream>>>(static_cast<const __half*>(x), scratch, rows, cols);
  else
    colsum_part_kernel<float><<<grid, 128, 0, stream>>>(static_cast<const float*>(x), scratch, rows, cols);
  colsum_final_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(scratch, out, parts, cols);
  return static_cast<int>(cudaGetLastError());
}
