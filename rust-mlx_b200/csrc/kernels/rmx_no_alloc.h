// A matrix product for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (d9beuD/rust-mlx has no CUDA code
// and lets its tensor library allocate whatever it needs).  It exists for hosts that use
// these kernels outside the engine and are not allowed to call cudaMalloc on the path
// where they need a product: code running inside someone else's memory pool with a fixed
// budget, a real-time loop that must not take the allocator's lock, or a plug-in that is
// handed its buffers and nothing else.  The ordinary entry point, rmx_gemm_tcgen05, asks
// its caller for scratch memory when it splits the reduction over several blocks; this one
// brings its own.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// The largest scratch the library holds per GPU: RMX_STATIC_SCRATCH_FLOATS floats of partial
// sums (8 MiB) and RMX_STATIC_SCRATCH_TILES counters.  Every GPU on which the library is
// loaded keeps this memory until the process ends, whether or not the entry point is used.
#define RMX_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define RMX_STATIC_SCRATCH_TILES 4096

// C[M, N] = A[M, K] . W[N, K]^T in bfloat16 with float accumulation; 1 <= M <= 64, K a multiple
// of 8, A and W 16-byte aligned with leading dimensions (in elements) that are multiples of 8.
// out_float != 0: C is float32, else bfloat16.  splits >= 1 slices of K share each tile of 128
// rows of W (0: the library chooses).  The caller passes inputs and the output only.
//
// Returns 0, or -1 with a message for rmx_last_error(): sizes outside the above, or a split
// whose partial sums (splits * MPAD * ceil(N / 128) * 128 floats, MPAD = 16, 32 or 64 for M up
// to 16, 32, 64) would not fit RMX_STATIC_SCRATCH_FLOATS, or N beyond
// RMX_STATIC_SCRATCH_TILES * 128.  It never calls cudaMalloc, cudaFree or any routine that
// allocates device memory.
//
// The first call on a device looks up the address of the library's scratch on that device
// (the device must be current); make that first call before any stream capture.  All calls
// share the one scratch area: two calls whose kernels may overlap on the GPU (different
// streams, or one graph replayed concurrently with itself) race with each other.  The
// counters are cleared on the stream at the start of every call, so a call that was cut
// short does not spoil the next.
int rmx_gemm_tcgen05_static(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                            int out_float, int splits, void* stream);

// 0 if the last rmx_gemm_tcgen05_static kernel on the current device completed, 3 if it gave up
// a bounded wait; synchronises the stream it is given.
int rmx_gemm_tcgen05_static_status(void* stream);

#ifdef __cplusplus
}
#endif
