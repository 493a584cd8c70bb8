// Column sum for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference library.
//
// Who needs it: code that runs where cudaMalloc / cudaFree are off limits or unsafe - inside
// a region being captured into a CUDA graph, in a callback or a thread that must not take
// the allocator's locks, in a process whose memory budget was fixed at start-up, or in a
// host program (for instance a LuaJIT script binding this library through its FFI) that has
// no allocator of its own to hand a workspace to the kernel.  The regular column-sum entry
// points need a scratch buffer whose size depends on the input and get it from an allocator;
// this one keeps its scratch in a fixed array inside the library.
//
// Contract:
//   * out[c] = sum over r of in[r * ld + c], fp32 in / fp32 out, rows summed in a fixed
//     order (results are reproducible).
//   * No cudaMalloc, cudaFree or any allocating library call is made, on any call.
//   * The scratch is a file-scope device array of LT_NOALLOC_MAX_SCRATCH_FLOATS floats
//     (4 MiB).  Every GPU that loads the library holds those 4 MiB until the process exits.
//     A problem needs ceil(rows / 128) * cols scratch floats; larger problems are refused
//     with LT_NOALLOC_TOO_LARGE and a message on stderr, nothing is launched.
//   * The first call on a device looks up the device address of the scratch array (with that
//     device current).  Make that first call outside any stream capture.
//     The same answer is given for more than 65535 slabs of 128 rows (the launch grid's
//     limit).  rows == 0 writes zeros and uses no scratch.
//   * All calls share the one array: two calls whose kernels can overlap on the GPU
//     (different streams, no dependency between them) race on it.  They also share, with
//     EVERY other column sum of this library (the regular entry points and the bias-gradient
//     sums inside a training step included), the per-column-group ticket words that elect
//     the block which adds up the partial sums: a call that overlaps any other column sum on
//     another stream can corrupt both results.  Order them on one stream or with events.
//     The array keeps whatever the last call left in it; the kernels write every scratch
//     element they later read, so no clearing is needed between calls.
//   * The first call on a device is safe from several host threads at once (a mutex guards
//     the address lookup).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LT_NOALLOC_MAX_SCRATCH_FLOATS (1 << 20)

enum {
  LT_NOALLOC_OK = 0,
  LT_NOALLOC_BAD_ARGUMENT = 1,
  LT_NOALLOC_TOO_LARGE = 2,
  LT_NOALLOC_CUDA_ERROR = 3,
};

// `stream` is a cudaStream_t (pass 0 / NULL for the default stream).  Returns one of the
// codes above; the launch is asynchronous.
int lt_column_sum_f32_noalloc(const float* in, int64_t rows, int64_t cols, int64_t ld, float* out,
                              void* stream);

// Scratch floats the call above would need for this shape (to test against the maximum).
int64_t lt_column_sum_noalloc_scratch_floats(int64_t rows, int64_t cols);

#ifdef __cplusplus
}
#endif
