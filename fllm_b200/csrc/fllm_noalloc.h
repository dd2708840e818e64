// C entry point for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference engine. It exists for hosts that
// embed the kernels from plain C/C++ (no torch, no caching allocator) inside a serving
// process whose device memory is already fully handed out - typically to the paged KV
// pool, sized to a fraction of HBM at start-up. In such a process a cudaMalloc at request
// time can fail outright, and even when it succeeds it synchronises the whole device and
// stalls every other stream. So the split-K GEMM is offered here with its fp32 partial-sum
// scratch living in a fixed array inside the library image instead of a caller- or
// allocator-provided workspace.
//
//   y[tokens, features] = x[tokens, k] * w[features, k]^T (+ bias[features]), bf16 in/out,
//   computed as `splits` partial products over slices of k that are summed in fp32.
//
// Contract
//   * The caller passes inputs and outputs only (device pointers, leading dimensions in
//     elements, a CUDA stream). Nothing is allocated or freed: no cudaMalloc / cudaFree and
//     no allocating library routine is called, on any path.
//   * The scratch array is FLLM_NOALLOC_SCRATCH_BYTES (8 MiB) per device; every GPU on which
//     the library is loaded holds it until the process exits. A call needs 64 KiB (per-tile
//     arrival counters) + splits * tokens' * features' * 4 bytes of it, where tokens' is tokens
//     rounded up to 16 / 32 / 64 / a multiple of 128 and features' is features rounded up to a
//     multiple of 128; a call that needs more is rejected with FLLM_NOALLOC_E_TOO_LARGE and a
//     message naming both numbers (nothing is launched).
//   * Per-device set-up happens in fllm_noalloc_init(), or inside the first GEMM call on a device
//     if init was never called there: it looks up the device address of the scratch array (with
//     that device current) and sets the kernels' attributes. With CUDA's default lazy module
//     loading this is also the moment the driver materialises the kernels and the 8 MiB array on
//     that device, which takes device memory once. So run it at start-up - BEFORE the rest of the
//     memory is handed to the KV pool, and outside any stream capture; after it, calls take no
//     device memory at all.
//   * All calls on a device share the one array and it keeps whatever the previous call left
//     there. Only the arrival counters must be zero between calls, and every call leaves them at
//     zero again; the partial sums need no clearing because each call overwrites all it reads.
//     Two calls that overlap on the GPU (different streams, no ordering between them) would
//     race on the array - order them on one stream or with events.
//   * k, features and the leading dimensions must be multiples of 8; x, w and y must be 16-byte
//     aligned (checked: FLLM_NOALLOC_E_ARGS).
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FLLM_NOALLOC_SCRATCH_BYTES (8u << 20)

enum {
  FLLM_NOALLOC_OK = 0,
  FLLM_NOALLOC_E_ARGS = -1,       // null pointer, non-positive size, bad alignment or multiple
  FLLM_NOALLOC_E_TOO_LARGE = -2,  // 64 KiB of counters + splits * padded tokens * padded features * 4 exceeds the array
  FLLM_NOALLOC_E_CUDA = -3,       // a CUDA call failed (symbol lookup, launch)
};

// `stream` is a cudaStream_t (0 = default stream). `status` may be null; when given it is a
// device int that receives a non-zero code if a pipeline wait inside the kernel ran out.
// Returns FLLM_NOALLOC_OK or one of the negative codes above.
int fllm_linear_bf16_splitk_noalloc(const void* x, long long ldx, const void* w, long long ldw,
                                    const void* bias, void* y, long long ldy, int tokens,
                                    int features, int k, int splits, int* status, void* stream);

// Per-device set-up for the current device (see the contract above). Idempotent; returns
// FLLM_NOALLOC_OK or FLLM_NOALLOC_E_CUDA.
int fllm_noalloc_init(void);

// Message of the most recent failure on the calling thread ("" if none).
const char* fllm_noalloc_last_error(void);

// Size of the per-device scratch array, for callers that size their calls at run time.
size_t fllm_noalloc_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
