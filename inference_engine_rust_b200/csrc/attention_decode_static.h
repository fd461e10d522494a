// Split-KV decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference engine (which is CPU code with one
// heap-allocated cache per layer); it exists for hosts of this library that run inside a
// fixed memory budget: a process whose device memory was carved up once at start-up by
// another allocator, a plugin called from inside a region where cudaMalloc is forbidden or
// would synchronise the device, or a latency-critical loop that may not touch the driver's
// allocator at all.  Such callers cannot hand the kernel the scratch buffer that
// `iert_attention_decode` asks for, so this variant keeps the scratch in a fixed array that
// is part of the library image itself.
//
// What it does is exactly what `iert_attention_decode` does (same kernels, same arguments,
// same results); only the home of the partial results differs.
//
// Rules for the caller
//   * The caller still owns every input and the output: `qkv`, `out`, the batch arrays and the
//     cache behind `cache` are its memory.
//   * The scratch array holds IERT_STATIC_SCRATCH_FLOATS floats (8 MiB).  Every GPU that loads
//     the library carries this array from the moment the library's code is loaded on it until
//     the process exits, whether or not this function is ever called.
//   * A call needs n_tokens * heads * splits * (head_dim + 2) floats.  A call that needs more
//     is refused with IERT_STATIC_SCRATCH_TOO_SMALL and launches nothing; ask for fewer splits
//     or use `iert_attention_decode` with a buffer of your own.
//   * The first call on each device looks up the array's device address (with that device
//     current) and remembers it.  Make that first call outside any stream capture.  It may also
//     be the moment at which the CUDA runtime loads this library's code, the 8 MiB array
//     included, onto the device (module loading is lazy by default), so device memory in use can
//     still grow during that one call: a host that must not see that later makes one call at
//     start-up.  From the second call on nothing is loaded or looked up.
//   * All calls on one device share the one array.  Nothing in it has to be cleared between
//     calls, because every element a call reads was written earlier in the same call; but two
//     calls whose kernels can overlap on the GPU (different streams without an ordering
//     between them) race on it.  Order such calls yourself.
//   * Neither this function nor the kernels it launches call cudaMalloc, cudaFree or any
//     routine that allocates.
#pragma once

#include "common.cuh"

#define IERT_STATIC_SCRATCH_FLOATS (2u * 1024u * 1024u)

// Returned in addition to the common status codes.
enum : int {
  IERT_STATIC_SCRATCH_TOO_SMALL = 3,   // the call needs more scratch than the fixed array holds
  IERT_STATIC_SETUP_FAILED = 4,        // the array's device address could not be obtained
};

// Same arguments as iert_attention_decode, minus the scratch pointer.
IERT_API int iert_attention_decode_static(const void* qkv, void* out, const IertBatchView* batch,
                                          const IertKvView* cache, int heads, float scale, int splits,
                                          int* err, cudaStream_t stream);

// Floats of scratch the fixed array holds (IERT_STATIC_SCRATCH_FLOATS), for callers that size
// their batches against it.
IERT_API long long iert_attention_decode_static_capacity();

// A sentence for each status code this entry point can return.
IERT_API const char* iert_attention_decode_static_message(int status);
