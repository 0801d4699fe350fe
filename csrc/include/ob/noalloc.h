// Allocation-free entry point of the library.  It has no counterpart in the reference
// project: it exists for callers that hold raw device pointers and are not allowed to
// allocate device memory when they call in -- code running between cudaStreamBeginCapture
// and cudaStreamEndCapture of their own, real-time loops that forbid cudaMalloc's implicit
// device synchronisation, or processes that run with a fixed memory budget where any pool
// growth is an error.  The regular `sum` operator takes its block partials from the caching
// pool, which may call cudaMalloc; this variant keeps them in a static device array instead.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest input accepted, in elements (1 Gi float32 values = 4 GiB).
#define ORTHON_NOALLOC_SUM_MAX_ELEMENTS (1LL << 30)
// Size of the static scratch array, in float32 values (4 KiB per GPU that loads the library,
// held until the process exits).
#define ORTHON_NOALLOC_SUM_SCRATCH_FLOATS 1024

// out[0] = sum(in[0 .. n)) in float32, computed on `stream` (a cudaStream_t, may be null for
// the default stream) of the CURRENT device.  `in` and `out` are device pointers supplied by
// the caller; nothing is allocated or freed, neither by the CUDA runtime nor by any library.
//
// Return value: 0 on success; 1 for a null pointer or negative n; 2 when n exceeds
// ORTHON_NOALLOC_SUM_MAX_ELEMENTS; 3 when a CUDA call failed.  When `err` is not null a
// NUL-terminated description of the failure is written to it (at most `err_cap` bytes).
//
// The first call on each device looks up the address of the static scratch array (one
// cudaGetSymbolAddress, no allocation).  Make that first call before starting any stream
// capture on the device.
//
// All calls share the one scratch array, which keeps the partial sums of the most recent
// call; every call overwrites exactly the slots it later reads, so stale contents are never
// consumed.  Two calls that may run at the same time on one device (different streams, or
// different host threads) race on the array: serialise them.
int orthon_sum_f32_noalloc(const float* in, long long n, float* out, void* stream, char* err, unsigned long err_cap);

#ifdef __cplusplus
}
#endif
