// gesso_argmax_rows_static: greedy token selection that allocates nothing.
//
// This entry point has no counterpart in the reference; it exists for hosts that must not allocate
// device memory at the moment they select tokens.  Examples: a serving loop that has handed every
// free byte of the device to its own memory pool and forbids cudaMalloc afterwards (a fresh
// allocation would fail, or would stall every stream while the driver maps it); a plug-in called
// from inside another framework's step, where allocating through that framework's allocator is not
// possible from C; a caller with a latency budget that a driver allocation would break.  The
// regular entry point, gesso_argmax_rows, needs scratch memory from its caller for rows of 8192
// logits or more; this one carries its scratch inside the library instead.
//
// What it does: for each row of `logits` ([n_rows, vocab] float32, row-major, on the current
// device) writes the index of the largest value to ids[row] (ties go to the lowest index) and 1 or
// 0 to nonfinite[row] (1 if the row holds a NaN or an infinity; no token may be emitted then).  The
// result is the same as gesso_argmax_rows gives.
//
// Limits and rules:
//   * n_rows <= GESSO_ARGMAX_STATIC_MAX_ROWS (256).  More rows are refused with
//     GESSO_ARGMAX_STATIC_TOO_MANY_ROWS and nothing is launched.  vocab >= 1.
//   * The scratch is one fixed array of GESSO_ARGMAX_STATIC_SCRATCH_BYTES (96 KiB) of device
//     memory per GPU that loads this library, held until the process exits.
//   * The first call on each device looks up the array's device address (one runtime query, no
//     allocation).  Make that first call outside any stream capture; later calls only launch.
//   * All calls on a device share the array.  Nothing in it has to be zero at the start: every
//     call overwrites the part it reads.  Two calls that overlap in time on one device (different
//     streams, or two threads) would overwrite each other's partial results: issue them on one
//     stream, or otherwise order them.
//   * Nothing is allocated or freed: no cudaMalloc, no cudaFree, no library call that allocates.
//
// Returns 0, a negative refusal code below, or a positive cudaError_t from the set-up or the launch.
#pragma once
#include <cuda_runtime.h>

#define GESSO_ARGMAX_STATIC_MAX_ROWS 256
#define GESSO_ARGMAX_STATIC_SPLIT 32
#define GESSO_ARGMAX_STATIC_SCRATCH_BYTES (GESSO_ARGMAX_STATIC_MAX_ROWS * GESSO_ARGMAX_STATIC_SPLIT * 12)

#define GESSO_ARGMAX_STATIC_TOO_MANY_ROWS (-10)
#define GESSO_ARGMAX_STATIC_BAD_ARGUMENT (-11)

#ifdef __cplusplus
extern "C" {
#endif
__attribute__((visibility("default"))) int gesso_argmax_rows_static(const float* logits, int n_rows, int vocab,
                                                                    int* ids, int* nonfinite, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
