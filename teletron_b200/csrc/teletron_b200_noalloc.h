/* An entry point of libteletron_b200.so that allocates nothing.  It has no counterpart in the reference
 * (TeleTron's extensions allocate their temporaries with at::empty, teletron_op/fused_rmsnorm/weight_backward.cu:229).
 *
 * Who needs it: hosts that hand this library raw device pointers but must not, or cannot, obtain device memory
 * while the call runs - a C or C++ program that carved up the whole GPU at start-up, a plugin living inside another
 * runtime's fixed memory pool, code running where the allocator is frozen.  tt_rmsnorm_bwd expects such a caller to
 * bring a scratch buffer for the per-block column sums; tt_rmsnorm_bwd_noalloc brings its own.
 *
 * The scratch is a file-scope __device__ array inside the library (TT_NOALLOC_MAX_BLOCKS x TT_NOALLOC_MAX_COLS
 * floats = 2 MiB), present on every GPU that loads the library for the life of the process.  Consequences:
 *   - cols must be a multiple of 8 and at most TT_NOALLOC_MAX_COLS; larger requests return TT_ERR_LIMIT (4).
 *     Any row count is accepted.
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current).  Make that first call outside any stream capture.
 *   - all calls on a device share the one array.  Each call overwrites the part it reads, so calls issued one after
 *     another on a stream are independent, but two calls that can overlap on the GPU (different streams, no
 *     dependency) race on the array and must be serialised by the caller.
 *   - no cudaMalloc, cudaFree or any allocating library routine is called; inputs and outputs are the caller's.
 *
 * Arguments are those of tt_rmsnorm_bwd without `partials`: dy, x [rows, cols] bf16; w [cols] bf16; rstd [rows]
 * fp32 (from tt_rmsnorm_fwd); dx [rows, cols] bf16 out; dw [cols] bf16 out; stream is a cudaStream_t.
 * Returns TT_OK (0) or a TT_ERR_* code. */
#pragma once

#define TT_NOALLOC_MAX_BLOCKS 512
#define TT_NOALLOC_MAX_COLS 1024

#ifdef __cplusplus
extern "C" {
#endif

int tt_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx, void* dw,
                           long rows, int cols, void* stream);

#ifdef __cplusplus
}
#endif
