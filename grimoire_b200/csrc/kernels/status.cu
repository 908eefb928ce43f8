// Per-device status block written by kernels whose bounded waits ran out, read by the host.
// Layout: [0] first error code (GrmStatusCode, 0 = none), [1] detail word of that first error,
// [2] number of errors recorded, [3..7] reserved.
#include "common.cuh"

namespace {
__device__ unsigned int g_status_words[8];
int g_pdl = 6;
}

// Programmatic dependent launch of the decode kernels (see common.cuh): a mask of GRM_PDL_* bits, 0 = plain launches.
GRM_API void grm_set_pdl(int mask) { g_pdl = mask; }
GRM_API int grm_pdl_enabled() { return g_pdl; }

// Device address of the status block of the current device (resolved once per device).
GRM_API unsigned int* grm_status_ptr() {
  static unsigned int* cache[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_words) != cudaSuccess) return nullptr;
    cache[dev] = (unsigned int*)p;
  }
  return cache[dev];
}

// Copies the 8 status words to `out` (host) and optionally clears them.  Synchronises the stream.
GRM_API int grm_status_read(unsigned int* out, int clear, void* stream) {
  unsigned int* p = grm_status_ptr();
  if (!p) return (int)cudaErrorInvalidDevice;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(out, p, 8 * sizeof(unsigned int), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return (int)e;
  if (clear) {
    e = cudaMemsetAsync(p, 0, 8 * sizeof(unsigned int), st);
    if (e != cudaSuccess) return (int)e;
  }
  return (int)cudaStreamSynchronize(st);
}
