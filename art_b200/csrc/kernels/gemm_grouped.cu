// Grouped (mixture-of-experts) bf16 GEMM on the tcgen05 pipeline:
//
//   C[rows of expert e, :N] = A[rows of expert e, :K] * B_e[N, K]^T (+ A2[rows, :K2] * B2_e[N, K2]^T)
//
// Rows of A are sorted by expert, each expert's segment padded to a multiple of 128 rows, and a
// device array maps every 128-row tile to its expert, so one persistent launch covers all experts
// without the host knowing the (data-dependent) segment sizes.  B / B2 are the experts' matrices
// stacked along rows ([E * N, K]); the tile scheduler adds e * N to the TMA row coordinate.  The
// extra-K pair carries the per-expert LoRA update exactly as in the dense GEMM; the SwiGLU
// epilogue serves the gate|up projection.
//
// The reference supports dense models only (README "Supported models"); this kernel serves the
// sparse-expert configuration of the benchmark suite.  Unfused equivalent: a loop of library GEMMs
// over experts, or torch._grouped_mm.
#include "gemm_epilogue.cuh"
#include "host_utils.h"

namespace artb {

template <int BN, int STAGES>
static int launch_grouped(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2, const CUtensorMap& tB2,
                          int kb_main, int kb_extra, const SchedGrouped& sched, const EpiGrouped<BN>& epi, int* status,
                          cudaStream_t stream) {
  using L = GemmSmemLayout<BN, STAGES>;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, SchedGrouped, EpiGrouped<BN>, NoComm>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  int grid = sched.m_tiles * sched.n_tiles;
  if (grid > sm_count()) grid = sm_count();
  kern<<<grid, GEMM_THREADS, L::TOTAL, stream>>>(tA, tB, tA2, tB2, kb_main, kb_extra, sched, epi, status, NoComm{});
  return static_cast<int>(cudaGetLastError());
}

}  // namespace artb

using namespace artb;

// A [m_tiles*128, K]; B [E*N, K]; A2 [m_tiles*128, K2]; B2 [E*N, K2]; C [m_tiles*128, N] bf16;
// H [m_tiles*128, N/2] for EPI_SWIGLU; tile_expert int32 [m_tiles] on the device.
ARTB_EXPORT int artb_gemm_grouped_bf16_tn(const void* A, int lda, const void* B, int ldb, const void* A2, int lda2,
                                          const void* B2, int ldb2, int K2, void* C, int ldc, void* H, int ldh,
                                          const int* tile_expert, int m_tiles, int num_experts, int N, int K,
                                          int epilogue, int* status, cudaStream_t stream) {
  if (m_tiles <= 0 || num_experts <= 0 || N <= 0 || K <= 0 || K2 < 0) return ERR_BAD_SHAPE;
  if ((K & 7) || (K2 & 7) || (N & 7) || (ldc & 7)) return ERR_BAD_SHAPE;
  if (epilogue != EPI_BF16 && epilogue != EPI_SWIGLU) return ERR_BAD_SHAPE;
  if (epilogue == EPI_SWIGLU && (!H || (ldh & 7) || (N & 31))) return ERR_BAD_ALIGN;
  if (epilogue != EPI_SWIGLU) H = nullptr;
  const int M = m_tiles * GEMM_BM;
  const int bn = N >= 256 ? 256 : (N > 64 ? 128 : 64);
  CUtensorMap tA, tB, tA2, tB2;
  int e;
  if ((e = make_tmap_bf16_2d(&tA, A, M, K, lda, GEMM_BM, GEMM_BK))) return e;
  if ((e = make_tmap_bf16_2d(&tB, B, static_cast<uint64_t>(num_experts) * N, K, ldb, bn, GEMM_BK))) return e;
  if (K2 > 0) {
    if ((e = make_tmap_bf16_2d(&tA2, A2, M, K2, lda2, GEMM_BM, GEMM_BK))) return e;
    if ((e = make_tmap_bf16_2d(&tB2, B2, static_cast<uint64_t>(num_experts) * N, K2, ldb2, bn, GEMM_BK))) return e;
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  const int kb_main = (K + GEMM_BK - 1) / GEMM_BK, kb_extra = (K2 + GEMM_BK - 1) / GEMM_BK;
#define ARTB_LAUNCH(BN_, ST_)                                                                                  \
  {                                                                                                            \
    SchedGrouped sched{tile_expert, m_tiles, (N + BN_ - 1) / BN_, N};                                          \
    EpiGrouped<BN_> epi{EpiStore<BN_, 1>{C, nullptr, reinterpret_cast<__nv_bfloat16*>(H), nullptr, ldc, 0, ldh,   \
                                      M, N, 0, N}};                                                            \
    return launch_grouped<BN_, ST_>(tA, tB, tA2, tB2, kb_main, kb_extra, sched, epi, status, stream);          \
  }
  if (bn == 256) ARTB_LAUNCH(256, 4)
  if (bn == 128) ARTB_LAUNCH(128, 6)
  ARTB_LAUNCH(64, 8)
#undef ARTB_LAUNCH
}
