// Split-K tcgen05 GEMM for small-M (decode) shapes.
//
// With M <= 256 rows a projection is a weight-streaming problem: the useful traffic is the
// weight matrix, and what has to be avoided is re-reading the activation panel once per N tile.
// Wide N tiles (256) keep that re-read small but leave too few tiles to fill 148 SMs, so the K
// dimension is split as well: CTA (m_blk, n_blk, k_split) accumulates its K slice in TMEM and adds
// the 128 x BN partial into an fp32 workspace with vector atomics; a finalize pass adds bias /
// residual, rounds to bf16 and re-zeroes the workspace for the next call.
//
// Serves the decode-time projections of the rollout engine (the reference delegates these to
// its third-party engine's GEMMs: src/art/local/vllm.py:46-53).
#include "gemm_epilogue.cuh"
#include "host_utils.h"

namespace artb {

template <int BN, int STAGES>
static int launch_splitk(const CUtensorMap& tA, const CUtensorMap& tB, int kb_main, int M, int N, int splits,
                         float* ws, int ldw, int* status, cudaStream_t stream) {
  using L = GemmSmemLayout<BN, STAGES>;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, SchedSplitK, EpiAtomic<BN>>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  SchedSplitK sched;
  sched.m_tiles = (M + GEMM_BM - 1) / GEMM_BM;
  sched.n_tiles = (N + BN - 1) / BN;
  sched.splits = splits;
  sched.kb_per = (kb_main + splits - 1) / splits;
  sched.kb_main = kb_main;
  int grid = sched.m_tiles * sched.n_tiles * splits;
  if (grid > sm_count()) grid = sm_count();
  EpiAtomic<BN> epi{ws, ldw, M, N};
  return static_cast<int>(launch_kernel(kern, dim3(grid), dim3(GEMM_THREADS), L::TOTAL, stream, tA, tB, tA, tB, kb_main, 0,
                                        sched, epi, status, NoComm{}));
}

// out = bf16(ws + bias + residual[:, :res_cols]); ws <- 0.
// With `adapter`: columns >= mask_col0 hold the stacked LoRA shrink products of all resident adapters (`cols` per
// slot); row m keeps only the columns of its own slot adapter[m] (none if negative) -- the multi-LoRA slot mask,
// applied here so that it costs no launch of its own.
__global__ void splitk_finalize_kernel(float* __restrict__ ws, int ldw, __nv_bfloat16* __restrict__ out, int ldc,
                                       const __nv_bfloat16* __restrict__ R, int ldr, int res_cols,
                                       const float* __restrict__ bias, int M, int N, const int* __restrict__ adapter,
                                       int mask_col0, int cols) {
  pdl_wait();
  pdl_launch_dependents();
  const int vec = N >> 2;
  const long total = static_cast<long>(M) * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int m = i / vec, c = (i % vec) * 4;
    float4* w = reinterpret_cast<float4*>(ws + static_cast<size_t>(m) * ldw + c);
    float4 v = *w;
    *w = make_float4(0.f, 0.f, 0.f, 0.f);
    if (bias) {
      v.x += bias[c];
      v.y += bias[c + 1];
      v.z += bias[c + 2];
      v.w += bias[c + 3];
    }
    if (R && c < res_cols) {
      const __nv_bfloat16* r = R + static_cast<size_t>(m) * ldr + c;
      v.x += __bfloat162float(r[0]);
      v.y += __bfloat162float(r[1]);
      v.z += __bfloat162float(r[2]);
      v.w += __bfloat162float(r[3]);
    }
    if (adapter && c + 4 > mask_col0) {
      const int a = adapter[m];
      const int lo = mask_col0 + a * cols, hi = lo + cols;
      if (c >= mask_col0 && (a < 0 || c < lo || c >= hi)) v.x = 0.f;
      if (c + 1 >= mask_col0 && (a < 0 || c + 1 < lo || c + 1 >= hi)) v.y = 0.f;
      if (c + 2 >= mask_col0 && (a < 0 || c + 2 < lo || c + 2 >= hi)) v.z = 0.f;
      if (c + 3 >= mask_col0 && (a < 0 || c + 3 < lo || c + 3 >= hi)) v.w = 0.f;
    }
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(m) * ldc + c) = o;
  }
}

}  // namespace artb

using namespace artb;

// ws[M, ldw] (fp32, zero on entry) += A[M,K] B[N,K]^T, K split `splits` ways.  bn in {64,128,256}.
ARTB_EXPORT int artb_gemm_splitk_bf16_tn(const void* A, int lda, const void* B, int ldb, float* ws, int ldw, int M,
                                         int N, int K, int bn, int splits, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K & 7) || (N & 3) || (ldw & 3) || splits < 1) return ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(ws) & 15) return ERR_BAD_ALIGN;
  const int kb_main = (K + GEMM_BK - 1) / GEMM_BK;
  if (splits > kb_main) splits = kb_main;
  CUtensorMap tA, tB;
  int e;
  if ((e = make_tmap_bf16_2d(&tA, A, M, K, lda, GEMM_BM, GEMM_BK))) return e;
  if ((e = make_tmap_bf16_2d(&tB, B, N, K, ldb, bn, GEMM_BK))) return e;
  if (bn == 256) return launch_splitk<256, 4>(tA, tB, kb_main, M, N, splits, ws, ldw, status, stream);
  if (bn == 128) return launch_splitk<128, 6>(tA, tB, kb_main, M, N, splits, ws, ldw, status, stream);
  if (bn == 64) return launch_splitk<64, 8>(tA, tB, kb_main, M, N, splits, ws, ldw, status, stream);
  return ERR_BAD_SHAPE;
}

ARTB_EXPORT int artb_splitk_finalize(float* ws, int ldw, void* out, int ldc, const void* R, int ldr, int res_cols,
                                     const float* bias, int M, int N, const int* adapter, int mask_col0, int cols,
                                     cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((N & 3) || (ldc & 3) || (ldw & 3) || (R && (ldr & 1))) return ERR_BAD_SHAPE;
  long total = static_cast<long>(M) * (N / 4);
  long blocks = (total + 255) / 256;
  if (blocks > 148L * 8) blocks = 148L * 8;
  return static_cast<int>(launch_kernel(splitk_finalize_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, stream, ws,
                                        ldw, reinterpret_cast<__nv_bfloat16*>(out), ldc,
                                        reinterpret_cast<const __nv_bfloat16*>(R), ldr, res_cols > 0 ? res_cols : N,
                                        bias, M, N, adapter, mask_col0, cols));
}
