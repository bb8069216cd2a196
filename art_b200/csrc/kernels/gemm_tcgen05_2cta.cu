// bf16 TN GEMM on CTA pairs: C[M,N] = A[M,K] B[N,K]^T (+ A2 B2^T), 256 x 256 tiles computed by
// tcgen05.mma.cta_group::2 (see include/gemm_pipeline_2cta.cuh).  Same epilogues and argument
// conventions as artb_gemm_bf16_tn; used for the large training projections.
#include "gemm_epilogue.cuh"
#include "gemm_pipeline_2cta.cuh"
#include "host_utils.h"

namespace artb {

template <int STAGES, int BN2>
static int launch_2cta(const void* A, int lda, const void* B, int ldb, const void* A2, int lda2, const void* B2,
                       int ldb2, int K2, void* C, int ldc, const void* R, int ldr, void* H, int ldh, const float* bias,
                       int M, int N, int K, int epilogue, int res_cols, int* status, int max_clusters,
                       cudaStream_t stream) {
  using L = Gemm2SmemLayout<STAGES, BN2>;
  static_assert(L::TOTAL + 4 * EpiStore<BN2>::COL_SPLIT * 4096 + 64 <= 227 * 1024, "shared memory");
  CUtensorMap tA, tB, tA2, tB2;
  int e;
  if ((e = make_tmap_bf16_2d(&tA, A, M, K, lda, GEMM_BM, GEMM_BK))) return e;
  if ((e = make_tmap_bf16_2d(&tB, B, N, K, ldb, BN2 / 2, GEMM_BK))) return e;
  if (K2 > 0) {
    if ((e = make_tmap_bf16_2d(&tA2, A2, M, K2, lda2, GEMM_BM, GEMM_BK))) return e;
    if ((e = make_tmap_bf16_2d(&tB2, B2, N, K2, ldb2, BN2 / 2, GEMM_BK))) return e;
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  const int kb_main = (K + GEMM_BK - 1) / GEMM_BK, kb_extra = (K2 + GEMM_BK - 1) / GEMM_BK;
  auto kern = gemm_tcgen05_2cta_kernel<STAGES, BN2, SchedPair, EpiStore<BN2>>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    configured[dev & 63] = true;
  }
  const int m_tiles2 = (M + 2 * GEMM_BM - 1) / (2 * GEMM_BM), n_tiles = (N + BN2 - 1) / BN2;
  int clusters = m_tiles2 * n_tiles;
  int cap = sm_count() / 2;
  if (max_clusters > 0 && max_clusters < cap) cap = max_clusters;
  if (clusters > cap) clusters = cap;
  EpiStore<BN2> epi{C, reinterpret_cast<const __nv_bfloat16*>(R), reinterpret_cast<__nv_bfloat16*>(H), bias, ldc, ldr,
                      ldh, M, N, epilogue == EPI_F32 ? 1 : 0, res_cols > 0 ? res_cols : N,
                     epilogue == EPI_SWIGLU_BWD ? 1 : 0};
  SchedPair sched{m_tiles2, n_tiles, pick_group_m(m_tiles2, 2 * GEMM_BM, K), 1, kb_main, kb_main};
  return static_cast<int>(launch_kernel(kern, dim3(2 * clusters), dim3(gemm_pipe_threads<EpiStore<BN2>>()), L::TOTAL, stream,
                                        tA, tB, tA2, tB2, kb_main, kb_extra, sched, epi, status, NoComm{}));
}

// Split-K on CTA pairs for small-M (decode) weight streaming: work item = (256 x 256 tile, K slice); the pair shares
// each weight tile (every CTA stages half of it), so the weights cross L2 -> shared memory once per pair instead of
// once per 128-row tile, and the partial goes into the fp32 workspace with vector atomics.
static int launch_2cta_splitk(const void* A, int lda, const void* B, int ldb, float* ws, int ldw, int M, int N, int K,
                              int splits, int* status, cudaStream_t stream) {
  constexpr int STAGES = 6, BN2 = 256;
  using L = Gemm2SmemLayout<STAGES, BN2>;
  CUtensorMap tA, tB;
  int e;
  if ((e = make_tmap_bf16_2d(&tA, A, M, K, lda, GEMM_BM, GEMM_BK))) return e;
  if ((e = make_tmap_bf16_2d(&tB, B, N, K, ldb, BN2 / 2, GEMM_BK))) return e;
  const int kb_main = (K + GEMM_BK - 1) / GEMM_BK;
  if (splits > kb_main) splits = kb_main;
  const int kb_per = (kb_main + splits - 1) / splits;
  splits = (kb_main + kb_per - 1) / kb_per;   // no empty slice
  auto kern = gemm_tcgen05_2cta_kernel<STAGES, BN2, SchedPair, EpiAtomic<BN2>>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    configured[dev & 63] = true;
  }
  const int m_tiles2 = (M + 2 * GEMM_BM - 1) / (2 * GEMM_BM), n_tiles = (N + BN2 - 1) / BN2;
  int clusters = m_tiles2 * n_tiles * splits;
  if (clusters > sm_count() / 2) clusters = sm_count() / 2;
  EpiAtomic<BN2> epi{ws, ldw, M, N};
  SchedPair sched{m_tiles2, n_tiles, m_tiles2, splits, kb_per, kb_main};
  return static_cast<int>(launch_kernel(kern, dim3(2 * clusters), dim3(GEMM_THREADS), L::TOTAL, stream, tA, tB, tA, tB,
                                        kb_main, 0, sched, epi, status, NoComm{}));
}

}  // namespace artb

using namespace artb;

ARTB_EXPORT int artb_gemm_bf16_tn_2cta(const void* A, int lda, const void* B, int ldb, const void* A2, int lda2,
                                       const void* B2, int ldb2, int K2, void* C, int ldc, const void* R, int ldr,
                                       void* H, int ldh, const float* bias, int M, int N, int K, int epilogue,
                                       int res_cols, int* status, int max_clusters, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K2 < 0) return ERR_BAD_SHAPE;
  if ((K & 7) || (K2 & 7) || (N & 7)) return ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(C) & 15) return ERR_BAD_ALIGN;
  if (epilogue == EPI_F32 ? (ldc & 3) : (ldc & 7)) return ERR_BAD_ALIGN;
  if (epilogue != EPI_BF16_RESID && epilogue != EPI_SWIGLU) R = nullptr;
  if (epilogue != EPI_SWIGLU && epilogue != EPI_SWIGLU_BWD) H = nullptr;
  if (epilogue == EPI_BF16_RESID && (!R || (ldr & 7) || (reinterpret_cast<uintptr_t>(R) & 15))) return ERR_BAD_ALIGN;
  if ((epilogue == EPI_SWIGLU || epilogue == EPI_SWIGLU_BWD) && (!H || (ldh & 7) || (N & 31) || (reinterpret_cast<uintptr_t>(H) & 15)))
    return ERR_BAD_ALIGN;
  // 224-wide cluster tiles waste less of the last wave for some N (3584: 6.92 waves instead of 6.05) but
  // measured no faster under the power cap; they are kept for explicit requests (max_clusters < 0).
  if (max_clusters < 0)
    return launch_2cta<6, 224>(A, lda, B, ldb, A2, lda2, B2, ldb2, K2, C, ldc, R, ldr, H, ldh, bias, M, N, K, epilogue,
                               res_cols, status, -max_clusters, stream);
  return launch_2cta<6, 256>(A, lda, B, ldb, A2, lda2, B2, ldb2, K2, C, ldc, R, ldr, H, ldh, bias, M, N, K, epilogue,
                             res_cols, status, max_clusters, stream);
}

// ws[M, ldw] (fp32, zero on entry) += A[M,K] B[N,K]^T, K split `splits` ways over CTA pairs (256 x 256 tiles).
ARTB_EXPORT int artb_gemm_splitk_bf16_tn_2cta(const void* A, int lda, const void* B, int ldb, float* ws, int ldw, int M,
                                              int N, int K, int splits, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K & 7) || (N & 3) || (ldw & 3) || splits < 1) return ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(ws) & 15) return ERR_BAD_ALIGN;
  return launch_2cta_splitk(A, lda, B, ldb, ws, ldw, M, N, K, splits, status, stream);
}
