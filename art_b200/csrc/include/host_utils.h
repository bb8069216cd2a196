// Host-side helpers shared by the launchers: TMA tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda), cached device facts.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define ARTB_EXPORT extern "C" __attribute__((visibility("default")))

namespace artb {

// Error codes returned by the C entry points (cudaError_t values are positive).
enum HostError : int {
  ERR_BAD_SHAPE = -1,
  ERR_BAD_ALIGN = -2,
  ERR_NO_DRIVER = -3,
  ERR_TMAP = -4,
  ERR_TOO_LARGE = -5,
};

inline PFN_cuTensorMapEncodeTiled get_tmap_encoder() {
  static PFN_cuTensorMapEncodeTiled fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
    }
  }
  return fn;
}

// 2-D bf16 row-major tensor [rows, cols] with leading dimension ld (elements),
// tiled as boxes of [box_rows, box_cols]; box_cols * 2 B must be <= the swizzle span.
inline int make_tmap_bf16_2d(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                             uint64_t ld, uint32_t box_rows, uint32_t box_cols,
                             CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  auto enc = get_tmap_encoder();
  if (!enc) return ERR_NO_DRIVER;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * 2) & 15)) return ERR_BAD_ALIGN;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstr,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)   // say which descriptor was refused: the caller only sees ERR_TMAP
    fprintf(stderr, "artb: cuTensorMapEncodeTiled failed (%d): ptr=%p rows=%llu cols=%llu ld=%llu box=[%u x %u]\n",
            static_cast<int>(r), ptr, static_cast<unsigned long long>(rows), static_cast<unsigned long long>(cols),
            static_cast<unsigned long long>(ld), box_rows, box_cols);
  return r == CUDA_SUCCESS ? 0 : ERR_TMAP;
}

// Programmatic dependent launch.  While the switch is on (the rollout engine turns it on around its decode step), the
// launchers below mark their kernels as allowed to start before the previous kernel of the stream has finished; every
// such kernel executes `griddepcontrol.wait` (pdl_wait() in device code) before its first access to global memory, so
// only its prologue (barrier / TMEM setup, descriptor prefetch, block scheduling) overlaps the predecessor's tail.  A
// decode step is ~230 short launches whose hand-over gaps add up to a fifth of the step.  Kernels launched without
// the attribute (everything while the switch is off, and all library kernels) keep full stream order.
inline int& pdl_switch() {
  static int on = 0;
  return on;
}

template <class... KArgs, class... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_switch() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

inline int sm_count() {
  static int n[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!n[dev]) cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
  return n[dev];
}

}  // namespace artb
