// An attention entry point for callers that must not allocate device memory.
//
// This has no counterpart in the reference; it exists for users of this library.
//
// Some programs call into a kernel library from places where asking the CUDA
// allocator for memory is not an option: inside a real-time loop that may not
// block on the driver, from a host process that was handed a fixed memory budget
// and a ready-made set of buffers, or from a plug-in whose host owns the
// allocator and forbids foreign cudaMalloc calls.  The ordinary entry point
// jb_attention() needs the caller to bring a scratch buffer for the partial
// softmax results; whoever cannot allocate one can call jb_attention_noalloc()
// instead.  It runs the same two kernels, but keeps the partial results in a
// fixed array that is part of the library's device image.
//
// What a caller has to know:
//
// * The array is JB_NOALLOC_SCRATCH_FLOATS floats (32 MiB).  Every GPU on which
//   the library is loaded holds that much until the process exits, whether or
//   not this function is ever called.
// * A call needs jb_attention_scratch(n_rows, nh, hd, max_chunks) floats.  When
//   that exceeds the array, nothing is launched and JB_ETOOBIG is returned;
//   jb_attention_noalloc_error() then says how many floats were wanted.  Call
//   again with fewer rows (rows are independent; row0 / n_rows select them).
// * The first call on a device looks up the array's device address
//   (cudaGetSymbolAddress) with that device current, and remembers it.  Make
//   this first call before any stream capture starts on that device.
// * The function itself calls no cudaMalloc, cudaFree or other allocating
//   routine, neither directly nor through a library.
// * All calls on a device share the one array, and it keeps what the last call
//   left in it.  Nothing in it has to be zero beforehand: every partial result
//   that the merge step reads has been written by the same call.  Two calls
//   whose kernels can overlap on the GPU (different streams, no ordering between
//   them) race on the array and give wrong results; order them.
// * Threads: the address found at a device's first call is kept in a plain static
//   table without a lock.  Two threads that make a device's first call at the same
//   time both look the address up and both store the same value, which is harmless;
//   the calls themselves must be ordered anyway, as said above.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#define JB_NOALLOC_SCRATCH_FLOATS (8ll * 1024 * 1024)
#define JB_ETOOBIG (-3)   /* the call needs more scratch than the fixed array has */
#define JB_EDEVICE (-4)   /* the array's address could not be obtained on this device */

#ifdef __cplusplus
extern "C" {
#endif

/* Same arguments and results as jb_attention() (kernels.h), without the scratch
   pointer.  Returns 0, JB_EINVAL, JB_ELAUNCH, JB_ETOOBIG or JB_EDEVICE. */
int jb_attention_noalloc(const void *q, const void *k_cache, const void *v_cache, int dt,
                         const int32_t *row_pos, const int32_t *row_seq,
                         const int32_t *block_table, int bt_stride, void *out, int row0,
                         int n_rows, int nh, int nkv, int hd, int window, float scale,
                         int max_chunks, cudaStream_t st);

/* Why the last call on this thread failed, as text ("" after a success). */
const char *jb_attention_noalloc_error(void);

#ifdef __cplusplus
}
#endif
