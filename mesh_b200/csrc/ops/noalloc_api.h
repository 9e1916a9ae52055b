// RMSNorm backward for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for hosts of this library
// that are handed their buffers by someone else and own no allocator they are allowed to call:
// a plugin inside an inference server whose memory budget is fixed at start-up, a custom-call
// hook of another runtime that passes raw device pointers, or a process that has given all of
// its device memory to one arena and must not grow.  For them, mesh_rmsnorm_bwd is awkward
// because it wants a caller-provided fp32 scratch matrix for the per-block weight-gradient
// partials.  mesh_rmsnorm_bwd_noalloc needs inputs and outputs only: its partials live in a
// fixed array inside the library image.
//
// What that costs and what to watch for:
//   * The array is MESH_NOALLOC_MAX_BLOCKS x MESH_NOALLOC_MAX_COLS floats (4 MiB).  Every GPU
//     whose context loads the library holds that much until the process exits.
//   * cols must be a multiple of 8 and <= MESH_NOALLOC_MAX_COLS; anything else is refused with
//     an error text (mesh_last_error) and nothing is launched.
//   * The first call on each device looks up the array's device address (with that device
//     current) and remembers it.  Make that first call during set-up, before any stream capture.
//   * There is one array per device, shared by every call and every stream.  Two calls whose
//     kernels overlap on the GPU race on it: issue them on one stream, or order them yourself.
//     The array keeps whatever the previous call left; this op overwrites every element it later
//     reads, so nothing has to be cleared between calls.
//   * The function calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define MESH_NOALLOC_MAX_BLOCKS 128
#define MESH_NOALLOC_MAX_COLS 8192

// dx[rows, cols] (bf16) and dw[cols] (fp32) from dy, x (bf16 [rows, cols]), w (bf16 [cols]) and
// rstd (fp32 [rows], as written by mesh_rmsnorm_fwd).  Same math as mesh_rmsnorm_bwd.
// Returns 0, a negative argument error, or a positive cudaError_t.
int mesh_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw,
                             int rows, int cols, float w_offset, void* stream);

#ifdef __cplusplus
}
#endif
