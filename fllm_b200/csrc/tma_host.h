// Host-side helpers shared by the kernel launchers: tensor-map encoding through
// the driver entry point (so the library never links libcuda directly), SM count
// cache and error reporting.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdexcept>
#include <stdlib.h>
#include <utility>
#include <string>

namespace fllm {

inline void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    throw std::runtime_error(std::string("fllm_b200: ") + what + ": " + cudaGetErrorString(e));
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cuda_check(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q),
               "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    if (q != cudaDriverEntryPointSuccess || !p)
      throw std::runtime_error("fllm_b200: cuTensorMapEncodeTiled is not available");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows][cols] of `elem_bytes` elements with a row pitch of
// `pitch_bytes`; box = [box_rows][box_cols]; 128-byte swizzle (box_cols*elem_bytes
// must be 128) or none. Out-of-range elements read as zero.
inline CUtensorMap make_tmap_2d(const void* base, CUtensorMapDataType dt, int elem_bytes,
                                uint64_t rows, uint64_t cols, uint64_t pitch_bytes,
                                uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  CUtensorMap m;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15))
    throw std::runtime_error("fllm_b200: TMA operand must be 16-byte aligned with a 16-byte pitch");
  CUresult r = get_encode_tiled()(
      &m, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
      swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw std::runtime_error("fllm_b200: cuTensorMapEncodeTiled failed with code " +
                             std::to_string((int)r));
  (void)elem_bytes;
  return m;
}

// Programmatic dependent launch: the kernel may start while its predecessor in the stream is
// still running; it must execute griddepcontrol.wait before it touches anything the predecessor
// produces. FLLM_PDL=0 turns the attribute off (plain stream order).
inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("FLLM_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cuda_check(cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...), "cudaLaunchKernelEx");
}

// Same, with the grid cut into thread-block clusters of `cluster_x` consecutive CTAs.
template <typename... KArgs, typename... Args>
inline void launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               unsigned cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster_x;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cuda_check(cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...), "cudaLaunchKernelEx(cluster)");
}

// True the first time it is called on the current device for a given flag array: function attributes
// (dynamic shared-memory limits) are per device, so a process that drives several GPUs sets them on each.
// Use as  `static bool done[kMaxDevices] = {}; if (first_call_on_device(done)) { cudaFuncSetAttribute(...); }`
constexpr int kMaxDevices = 64;
inline bool first_call_on_device(bool (&done)[kMaxDevices]) {
  int dev = 0;
  cudaGetDevice(&dev);
  dev &= kMaxDevices - 1;
  if (done[dev]) return false;
  done[dev] = true;
  return true;
}

inline int sm_count() {
  static int n[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev];
}

}  // namespace fllm
