// Column sums without any allocation.
//
// This entry point has no counterpart in the reference package. It exists for callers that are not
// allowed to obtain device memory at the moment of the call: code holding a memory-pool lock, real-time or
// interrupt-style host threads where cudaMalloc's implicit device synchronisation is unacceptable, and
// embedders whose memory budget was fixed at start-up and who therefore hand a library nothing but input
// and output buffers. The ordinary `oslo_colsum`
// needs a [parts, cols] float workspace from its caller; here that workspace is a fixed array that lives in
// the library image itself.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest `cols` the built-in workspace can serve. The workspace is OSLO_NOALLOC_COLSUM_PARTS x
// OSLO_NOALLOC_COLSUM_MAX_COLS floats = 4 MiB, and every GPU that loads this library keeps those 4 MiB
// reserved until the process exits.
#define OSLO_NOALLOC_COLSUM_MAX_COLS 16384
#define OSLO_NOALLOC_COLSUM_PARTS 64

// out[c] = sum over r of x[r, c], accumulated in fp32.
//   x     : [rows, cols] row-major device buffer, dtype = OSLO_DT_BF16 / OSLO_DT_FP16 / OSLO_DT_FP32
//   out   : [cols] float device buffer
//   stream: stream of the CURRENT device to enqueue on
// Returns 0 on success; -2 unknown dtype; -3 bad pointer or negative size, and also a current-device index
// of 64 or more or a workspace whose address could not be resolved; -10 cols exceeds
// OSLO_NOALLOC_COLSUM_MAX_COLS (nothing is launched); a positive value is a cudaError_t. A launch error
// that an EARLIER, unrelated call left pending on this thread is returned (and cleared) before anything is
// launched, so that it is not mistaken for a failure of this call's kernels.
//
// Never calls cudaMalloc, cudaFree or any allocating routine. The first call on each device looks up the
// device address of the built-in workspace (cudaGetSymbolAddress) and remembers it; make that first call
// outside of any stream capture. All calls on one device share the one workspace: calls that may overlap on
// the GPU (different streams without an ordering between them) race on it and must be serialised by the
// caller. The workspace keeps whatever the previous call left in it; this routine overwrites every element
// it later reads, so nothing needs to be cleared between calls.
__attribute__((visibility("default")))
int oslo_colsum_noalloc(const void* x, float* out, int rows, int cols, int dtype, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
