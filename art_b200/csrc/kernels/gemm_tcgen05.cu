// bf16 GEMM  C[M,N] = A[M,K] * B[N,K]^T (+ A2[M,K2] * B2[N,K2]^T)  on tcgen05/TMEM,
// with fused epilogues.  Both operands are K-major ("TN"), which is how activations
// [tokens, features] and nn.Linear weights [out, in] are already laid out; the
// backward data-gradient uses a resident transposed copy of the frozen weight so
// that it is a TN GEMM as well.
//
// Epilogues (runtime-selected, applied per 32-column accumulator slab):
//   EPI_BF16        C = bf16(acc)
//   EPI_BF16_RESID  C = bf16(acc + R)                 residual add (o_proj / down_proj)
//   EPI_F32         C = acc                           fp32 output
//   EPI_SWIGLU      columns are interleaved in groups of 16 (gate | up):
//                   GU = bf16(acc) is stored [M, N] and H[M, N/2] = silu(gate) * up
//
// Covers the reference's cuBLAS-delegated projections (src/art/local/train.py:239-241
// runs the HF/Unsloth model whose q/k/v/o/gate/up/down projections are library GEMMs)
// and the PEFT LoRA branch, folded in as extra K.
#include "gemm_epilogue.cuh"
#include "host_utils.h"

namespace artb {

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2,
                       const CUtensorMap& tB2, int kb_main, int kb_extra, int M, int N,
                       const EpiStore<BN>& epi, int* status, int max_ctas, cudaStream_t stream) {
  using L = GemmSmemLayout<BN, STAGES>;
  // operand stages + the epilogue warps' 4 KB re-layout slabs (static shared memory) must fit the 227 KB of a CTA
  static_assert(L::TOTAL + 4 * EpiStore<BN>::COL_SPLIT * 4096 + 64 <= 227 * 1024, "shared memory");
  auto kern = gemm_tcgen05_kernel<BN, STAGES, SchedMFast, EpiStore<BN>>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  const int m_tiles = (M + GEMM_BM - 1) / GEMM_BM;
  SchedMFast sched{m_tiles, (N + BN - 1) / BN, pick_group_m(m_tiles, GEMM_BM, kb_main * GEMM_BK)};
  int grid = sched.m_tiles * sched.n_tiles;
  int cap = sm_count();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  return static_cast<int>(launch_kernel(kern, dim3(grid), dim3(gemm_pipe_threads<EpiStore<BN>>()), L::TOTAL, stream, tA, tB,
                                        tA2, tB2, kb_main, kb_extra, sched, epi, status, NoComm{}));
}

}  // namespace artb

using namespace artb;

// Tile width for an [M, N] output on `ctas` persistent CTAs: the widest tile that still fills the
// machine.  Narrower tiles that would waste less of the last wave (224 for N = 3584: 6.92 waves
// instead of 6.05) were measured and are no faster on a power-capped B200 (SMs idle in the last
// wave let the others clock higher), so 224 / 192 are only used on request.
ARTB_EXPORT int artb_pick_bn(int M, int N, int ctas) {
  const long m_tiles = (M + GEMM_BM - 1) / GEMM_BM;
  if (N >= 256 && m_tiles * ((N + 255) / 256) >= ctas) return 256;
  if (N >= 128 && m_tiles * ((N + 127) / 128) >= ctas / 2) return 128;
  return N > 64 ? 128 : 64;
}

// C[M,N] = A[M,K] B[N,K]^T (+ A2[M,K2] B2[N,K2]^T), bf16 inputs, fp32 accumulation in TMEM.
//   A, B, A2, B2 : bf16 row-major, leading dimensions in elements (multiples of 8), 16-B aligned
//   K2 == 0      : no extra-K operand (A2/B2 ignored)
//   epilogue     : GemmEpilogue (EPI_SWIGLU_BWD: H = forward gate|up [M,2N] input, C = d(gate|up) [M,2N] output); R (bf16 [M,res_cols]) is added for EPI_BF16_RESID and, when given, for EPI_SWIGLU;
//                  H (bf16 [M,N/2]) receives silu(gate)*up for EPI_SWIGLU;  res_cols 0 = all N columns
//   bias         : optional fp32 [N], added to the accumulator before any other epilogue step
//   bn           : tile width 64 / 128 / 192 / 224 / 256 (0 = choose, see artb_pick_bn)
//   status       : device int32, receives a KernelStatus on a bounded-wait expiry (0 otherwise)
//   max_ctas     : cap on the persistent grid (0 = one CTA per SM)
// Returns 0, a negative HostError, or a positive cudaError_t.
ARTB_EXPORT int artb_gemm_bf16_tn(const void* A, int lda, const void* B, int ldb, const void* A2,
                                  int lda2, const void* B2, int ldb2, int K2, void* C, int ldc,
                                  const void* R, int ldr, void* H, int ldh, const float* bias, int M,
                                  int N, int K, int epilogue, int res_cols, int bn, int* status, int max_ctas,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K2 < 0) return ERR_BAD_SHAPE;
  if ((K & 7) || (K2 & 7) || (N & 7)) return ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(C) & 15) return ERR_BAD_ALIGN;
  if (epilogue == EPI_F32 ? (ldc & 3) : (ldc & 7)) return ERR_BAD_ALIGN;
  if (epilogue != EPI_BF16_RESID && epilogue != EPI_SWIGLU) R = nullptr;
  if (epilogue != EPI_SWIGLU && epilogue != EPI_SWIGLU_BWD) H = nullptr;
  if (epilogue == EPI_BF16_RESID && (!R || (ldr & 7) || (reinterpret_cast<uintptr_t>(R) & 15)))
    return ERR_BAD_ALIGN;
  if ((epilogue == EPI_SWIGLU || epilogue == EPI_SWIGLU_BWD) && (!H || (ldh & 7) || (N & 31) || (reinterpret_cast<uintptr_t>(H) & 15)))
    return ERR_BAD_ALIGN;
  if (bn == 0) bn = artb_pick_bn(M, N, max_ctas > 0 && max_ctas < sm_count() ? max_ctas : sm_count());
  if (bn != 64 && bn != 128 && bn != 192 && bn != 224 && bn != 256) return ERR_BAD_SHAPE;

  CUtensorMap tA, tB, tA2, tB2;
  int e;
  if ((e = make_tmap_bf16_2d(&tA, A, M, K, lda, GEMM_BM, GEMM_BK))) return e;
  if ((e = make_tmap_bf16_2d(&tB, B, N, K, ldb, bn, GEMM_BK))) return e;
  if (K2 > 0) {
    if ((e = make_tmap_bf16_2d(&tA2, A2, M, K2, lda2, GEMM_BM, GEMM_BK))) return e;
    if ((e = make_tmap_bf16_2d(&tB2, B2, N, K2, ldb2, bn, GEMM_BK))) return e;
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  const int kb_main = (K + GEMM_BK - 1) / GEMM_BK;
  const int kb_extra = (K2 + GEMM_BK - 1) / GEMM_BK;

#define ARTB_LAUNCH(BN_, ST_)                                                                     \
  {                                                                                               \
    EpiStore<BN_> epi{C, reinterpret_cast<const __nv_bfloat16*>(R),                               \
                      reinterpret_cast<__nv_bfloat16*>(H), bias, ldc, ldr, ldh, M, N,              \
                      epilogue == EPI_F32 ? 1 : 0, res_cols > 0 ? res_cols : N,                   \
                      epilogue == EPI_SWIGLU_BWD ? 1 : 0};                                        \
    return launch_gemm<BN_, ST_>(tA, tB, tA2, tB2, kb_main, kb_extra, M, N, epi, status, max_ctas, \
                                 stream);                                                         \
  }
  if (bn == 256) ARTB_LAUNCH(256, 4)
  if (bn == 224) ARTB_LAUNCH(224, 4)
  if (bn == 192) ARTB_LAUNCH(192, 4)
  if (bn == 128) ARTB_LAUNCH(128, 6)
  ARTB_LAUNCH(64, 8)
#undef ARTB_LAUNCH
}
