// Exported C entry points of libkharon_cuda.so that are meant to be called directly by C/C++
// hosts (the Python package binds the full set through ctypes, see ops/_sigs.py).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

// Message of the last failed call on this thread (every entry point returns 0 or -1).
const char* kh_cuda_last_error(void);

// out[j] (+)= sum over rows of x[r, j]  for a bf16 matrix x [rows, N] with row pitch ld
// (elements), out fp32 [N], deterministic summation order.  `scratch` is caller-provided
// device memory of kh_colsum_scratch_elems(rows, N) floats, zeroed once before first use.
long kh_colsum_scratch_elems(int rows, int N);
int kh_colsum(const void* x, int ld, void* out, void* scratch, int rows, int N, int accumulate, void* stream);

// kh_colsum_noalloc -- the same column sum for hosts that are not allowed to allocate device
// memory at the point of the call.  (This entry point has no counterpart in the reference
// project; there every launcher may call cudaMalloc, e.g. flash.cu:201-229 allocates per call.)
//
// Who needs it: hosts whose device memory is fully partitioned at start-up and who may not grow
// it later, serving loops that must never take the driver's allocation lock (an allocation can
// synchronise the whole device), and plugins that are handed raw pointers but no allocator and
// must not mix a second allocator into the embedding application.  For them the
// partial sums and ticket counters that kh_colsum keeps in caller scratch live in a fixed array
// inside the library image instead: (1024 + 65536) floats = 266 240 bytes per GPU that loads the
// library, held until the process exits.  The call allocates and frees nothing, neither through
// the CUDA runtime nor through any library.
//
// Limits and rules:
//   * ceil(N / 64) <= 1024 and splits(rows, N) * N <= 65536 floats; larger problems are rejected
//     with -1 and a message naming the limit (use kh_colsum with your own scratch for those);
//   * x must be 16-byte aligned with ld a multiple of 8, like kh_colsum;
//   * the first call on each device looks up the array's device address (with that device
//     current); make that first call outside any stream capture;
//   * all calls on a device share the one array, and it keeps the previous call's contents (the
//     counters are cleared at the start of every call): two calls whose kernels can overlap on
//     the GPU -- different streams without an ordering between them -- race on it.  Order them.
int kh_colsum_noalloc(const void* x, int ld, void* out, int rows, int N, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
