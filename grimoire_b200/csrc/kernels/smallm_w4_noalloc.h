// grm_smallm_w4_noalloc -- the int4 small-M product (see smallm_w4.cu) for callers that cannot
// allocate device memory.  This entry point has no counterpart in the reference engine.
//
// Who needs it.  The ordinary entry point, grm_smallm_w4, takes its split-K scratch (per-slice
// partial sums and per-tile arrival counters) from the caller, and the Python layer gets that
// scratch from torch's allocator.  Some hosts of this library cannot do that: a process that gave
// the whole device to its own memory pool at start-up, so that a later cudaMalloc fails or
// fragments the pool; a latency-bound serving loop that may not take the device-wide
// synchronisation cudaMalloc / cudaFree can imply; a plug-in that is only handed input and output
// buffers and has no allocator of its own.  For them the scratch is a fixed array inside the
// library image.
//
// What it costs.  GRM_NOALLOC_MAX_PARTIAL_FLOATS floats (4 MiB) and GRM_NOALLOC_MAX_TILES counters
// (16 KiB) of device memory on every GPU that loads the library, held until the process exits,
// whether or not this function is ever called.
//
// Contract.
//  * Same arguments and results as grm_smallm_w4 minus the scratch / counters pointers; epi 0..3
//    (bf16 store, fp32 store, fp32 accumulate, SwiGLU).  The caller still owns w, sz, x and out.
//  * Split-K problems (ksplit > 1) whose scratch would not fit -- ksplit * (N / rows_per_cta) *
//    rows_per_cta/16 * roundup_pow2(ceil(M/8)) * 128 floats, or more than GRM_NOALLOC_MAX_TILES row
//    tiles -- are refused with GRM_NOALLOC_TOO_LARGE and nothing is launched.  With ksplit == 1 the
//    scratch is not touched and no size limit applies.
//  * It calls no cudaMalloc, cudaFree or allocating library routine.  The first call on a device
//    resolves the device addresses of the arrays (cudaGetSymbolAddress, with that device current);
//    make that first call before starting any stream capture.  That set-up is guarded (once per
//    device ordinal), so host threads may make their first calls concurrently; the calls themselves
//    still share the scratch, see the last point.
//  * Every call on a device uses the same arrays.  The counters are cleared at the start of each
//    call (on the caller's stream); the partial sums keep whatever the previous call left and are
//    fully rewritten before they are read.  Two calls that overlap on the GPU (different streams
//    without an ordering between them) race on this scratch and give wrong results: serialise them.
#pragma once

#define GRM_NOALLOC_MAX_PARTIAL_FLOATS (1 << 20)
#define GRM_NOALLOC_MAX_TILES 4096
#define GRM_NOALLOC_TOO_LARGE (-5)

#ifdef __cplusplus
extern "C" {
#endif

int grm_smallm_w4_noalloc(const void* w, const void* sz, const void* x, void* out, int M, int N, int K, int ldx, int ldo,
                          int group, int epi, int rows_per_cta, int ksplit, void* stream);

#ifdef __cplusplus
}
#endif
