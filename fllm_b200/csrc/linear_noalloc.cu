// Split-K bf16 GEMM behind a C entry point that allocates nothing: the fp32 partial sums
// go to a fixed array in this library's device image. See fllm_noalloc.h for the contract.
#include "fllm_noalloc.h"

#include <stdio.h>

#include <exception>
#include <mutex>

#include "fllm_ops.h"

#define FLLM_EXPORT extern "C" __attribute__((visibility("default")))

// The scratch itself. In host code this name is only a stand-in for the symbol: it is never
// passed to a kernel. The device address is looked up once per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[FLLM_NOALLOC_SCRATCH_BYTES];

// Keeps the array referenced from device code so the device linker cannot drop it.
__global__ void fllm_noalloc_scratch_anchor(unsigned long long* out) {
  if (out) *out = reinterpret_cast<unsigned long long>(&g_noalloc_scratch[0]);
}

namespace {

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;
thread_local char g_error[256] = "";

int fail(int code, const char* fmt, long long a = 0, long long b = 0) {
  snprintf(g_error, sizeof(g_error), fmt, a, b);
  return code;
}

// Device address of the scratch array on the current device (looked up on first use).
int scratch_for_current_device(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(FLLM_NOALLOC_E_CUDA, "cudaGetDevice failed with code %lld", (long long)e);
  if (dev < 0 || dev >= kMaxDevices)
    return fail(FLLM_NOALLOC_E_ARGS, "device ordinal %lld is outside the supported range [0, %lld)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return fail(FLLM_NOALLOC_E_CUDA, "cudaGetSymbolAddress(scratch) failed with code %lld on device %lld",
                  (long long)e, dev);
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return FLLM_NOALLOC_OK;
}

}  // namespace

FLLM_EXPORT size_t fllm_noalloc_scratch_bytes(void) { return FLLM_NOALLOC_SCRATCH_BYTES; }

FLLM_EXPORT const char* fllm_noalloc_last_error(void) { return g_error; }

FLLM_EXPORT int fllm_noalloc_init(void) {
  g_error[0] = 0;
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != FLLM_NOALLOC_OK) return rc;
  try {
    fllm::gemm_bf16_prepare_device();
  } catch (const std::exception& e) {
    snprintf(g_error, sizeof(g_error), "%s", e.what());
    return FLLM_NOALLOC_E_CUDA;
  }
  return FLLM_NOALLOC_OK;
}

FLLM_EXPORT int fllm_linear_bf16_splitk_noalloc(const void* x, long long ldx, const void* w, long long ldw,
                                                const void* bias, void* y, long long ldy, int tokens,
                                                int features, int k, int splits, int* status, void* stream) {
  g_error[0] = 0;
  if (!x || !w || !y) return fail(FLLM_NOALLOC_E_ARGS, "x, w and y must be non-null device pointers");
  if (tokens <= 0 || features <= 0 || k <= 0 || splits <= 0)
    return fail(FLLM_NOALLOC_E_ARGS, "tokens, features, k and splits must be positive");
  if ((k & 7) || (features & 7) || (ldx & 7) || (ldw & 7) || (ldy & 7))
    return fail(FLLM_NOALLOC_E_ARGS, "k, features and the leading dimensions must be multiples of 8");
  if ((reinterpret_cast<unsigned long long>(x) | reinterpret_cast<unsigned long long>(w) |
       reinterpret_cast<unsigned long long>(y)) & 15ull)
    return fail(FLLM_NOALLOC_E_ARGS, "x, w and y must be 16-byte aligned");
  if (splits > 16) return fail(FLLM_NOALLOC_E_ARGS, "splits must be at most 16 (got %lld)", splits);
  // partial sums are kept per tile: tokens round up to the tile width, features to 128; the first
  // 64 KiB of the array hold the per-tile arrival counters
  const unsigned long long tok_pad = tokens <= 16 ? 16 : tokens <= 32 ? 32 : tokens <= 64 ? 64
                                     : (unsigned long long)((tokens + 127) / 128) * 128;
  const unsigned long long feat_pad = (unsigned long long)((features + 127) / 128) * 128;
  const unsigned long long need = 65536ull + 4ull * (unsigned long long)splits * tok_pad * feat_pad;
  if (need > FLLM_NOALLOC_SCRATCH_BYTES)
    return fail(FLLM_NOALLOC_E_TOO_LARGE,
                "64 KiB + splits * padded tokens * padded features * 4 = %lld bytes exceeds the %lld-byte scratch array",
                (long long)need, (long long)FLLM_NOALLOC_SCRATCH_BYTES);
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != FLLM_NOALLOC_OK) return rc;
  try {
    fllm::linear_bf16(x, ldx, w, ldw, bias, y, ldy, tokens, features, k, scratch, FLLM_NOALLOC_SCRATCH_BYTES,
                      status, splits, static_cast<cudaStream_t>(stream));
  } catch (const std::exception& e) {
    snprintf(g_error, sizeof(g_error), "%s", e.what());
    return FLLM_NOALLOC_E_CUDA;
  }
  return FLLM_NOALLOC_OK;
}
