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
#include "gemm_pipeline.cuh"
#include "host_utils.h"

namespace artb {

enum GemmEpilogue : int { EPI_BF16 = 0, EPI_BF16_RESID = 1, EPI_F32 = 2, EPI_SWIGLU = 3 };

// Tiles are visited with the M index fastest, so the CTAs that run concurrently
// share a handful of weight (B) tiles and sweep the activation matrix, which
// stays L2-resident (M*K*2 bytes is tens of MB, L2 is 126 MB).
struct SchedMFast {
  int m_tiles, n_tiles;
  __device__ int tiles_for_cta(int cta, int ncta) const {
    const int total = m_tiles * n_tiles;
    return cta < total ? (total - cta + ncta - 1) / ncta : 0;
  }
  __device__ TileInfo get(int cta, int ncta, int i) const {
    const int t = cta + i * ncta;
    TileInfo ti;
    ti.m_blk = t % m_tiles;
    ti.n_blk = t / m_tiles;
    ti.first = ti.last = 1;
    ti.group = 0;
    return ti;
  }
};

template <int BN>
struct EpiStore {
  void* C;
  const __nv_bfloat16* R;
  __nv_bfloat16* H;  // SwiGLU output
  const float* bias;  // [N] fp32 or null
  int ldc, ldr, ldh;
  int M, N;
  int mode;

  __device__ void tile_begin(const TileInfo&, int) {}
  __device__ void tile_end(const TileInfo&, int) {}

  __device__ void chunk(const TileInfo& ti, int row, int c, uint32_t (&acc)[32]) {
    const int gr = ti.m_blk * GEMM_BM + row;
    const int gc = ti.n_blk * BN + c;
    if (gr >= M || gc >= N) return;
    const bool full = (gc + 32 <= N);
    if (bias) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (full || gc + j < N) acc[j] = __float_as_uint(__uint_as_float(acc[j]) + __ldg(bias + gc + j));
    }
    if (mode == EPI_F32) {
      float* out = reinterpret_cast<float*>(C) + static_cast<size_t>(gr) * ldc + gc;
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<uint4*>(out + j) = make_uint4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gc + j < N) out[j] = __uint_as_float(acc[j]);
      }
      return;
    }
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(C) + static_cast<size_t>(gr) * ldc + gc;
    if (mode == EPI_BF16_RESID) {
      const __nv_bfloat16* r = R + static_cast<size_t>(gr) * ldr + gc;
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 rv = *reinterpret_cast<const uint4*>(r + j);
          const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(rp[e]);
            acc[j + 2 * e] = __float_as_uint(__uint_as_float(acc[j + 2 * e]) + f.x);
            acc[j + 2 * e + 1] = __float_as_uint(__uint_as_float(acc[j + 2 * e + 1]) + f.y);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gc + j < N) acc[j] = __float_as_uint(__uint_as_float(acc[j]) + __bfloat162float(r[j]));
      }
    }
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1]));
        v.y = pack_bf16x2(__uint_as_float(acc[j + 2]), __uint_as_float(acc[j + 3]));
        v.z = pack_bf16x2(__uint_as_float(acc[j + 4]), __uint_as_float(acc[j + 5]));
        v.w = pack_bf16x2(__uint_as_float(acc[j + 6]), __uint_as_float(acc[j + 7]));
        *reinterpret_cast<uint4*>(out + j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (gc + j < N) out[j] = __float2bfloat16(__uint_as_float(acc[j]));
    }
    if (mode == EPI_SWIGLU && full) {
      // slab = [gate 0..15 | up 0..15]; the activation uses the bf16-rounded values so
      // that a backward pass that re-reads GU sees exactly what produced H.
      __nv_bfloat16* h = H + static_cast<size_t>(gr) * ldh + (gc >> 1);
      uint32_t hv[8];
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        float g0 = __bfloat162float(__float2bfloat16(__uint_as_float(acc[j])));
        float g1 = __bfloat162float(__float2bfloat16(__uint_as_float(acc[j + 1])));
        float u0 = __bfloat162float(__float2bfloat16(__uint_as_float(acc[16 + j])));
        float u1 = __bfloat162float(__float2bfloat16(__uint_as_float(acc[16 + j + 1])));
        float h0 = g0 / (1.f + __expf(-g0)) * u0;
        float h1 = g1 / (1.f + __expf(-g1)) * u1;
        hv[j >> 1] = pack_bf16x2(h0, h1);
      }
      *reinterpret_cast<uint4*>(h) = make_uint4(hv[0], hv[1], hv[2], hv[3]);
      *reinterpret_cast<uint4*>(h + 8) = make_uint4(hv[4], hv[5], hv[6], hv[7]);
    }
  }
};

template <int BN, int STAGES>
static int launch_gemm(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2,
                       const CUtensorMap& tB2, int kb_main, int kb_extra, int M, int N,
                       const EpiStore<BN>& epi, int* status, int max_ctas, cudaStream_t stream) {
  using L = GemmSmemLayout<BN, STAGES>;
  auto kern = gemm_tcgen05_kernel<BN, STAGES, SchedMFast, EpiStore<BN>>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  SchedMFast sched{(M + GEMM_BM - 1) / GEMM_BM, (N + BN - 1) / BN};
  int grid = sched.m_tiles * sched.n_tiles;
  int cap = sm_count();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  kern<<<grid, GEMM_THREADS, L::TOTAL, stream>>>(tA, tB, tA2, tB2, kb_main, kb_extra, sched, epi,
                                                 status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace artb

using namespace artb;

// C[M,N] = A[M,K] B[N,K]^T (+ A2[M,K2] B2[N,K2]^T), bf16 inputs, fp32 accumulation in TMEM.
//   A, B, A2, B2 : bf16 row-major, leading dimensions in elements (multiples of 8), 16-B aligned
//   K2 == 0      : no extra-K operand (A2/B2 ignored)
//   epilogue     : GemmEpilogue; R (bf16 [M,N]) for EPI_BF16_RESID; H (bf16 [M,N/2]) for EPI_SWIGLU
//   bias         : optional fp32 [N], added to the accumulator before any other epilogue step
//   bn           : tile width 64 / 128 / 256 (0 = choose)
//   status       : device int32, receives a KernelStatus on a bounded-wait expiry (0 otherwise)
//   max_ctas     : cap on the persistent grid (0 = one CTA per SM)
// Returns 0, a negative HostError, or a positive cudaError_t.
ARTB_EXPORT int artb_gemm_bf16_tn(const void* A, int lda, const void* B, int ldb, const void* A2,
                                  int lda2, const void* B2, int ldb2, int K2, void* C, int ldc,
                                  const void* R, int ldr, void* H, int ldh, const float* bias, int M,
                                  int N, int K, int epilogue, int bn, int* status, int max_ctas,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K2 < 0) return ERR_BAD_SHAPE;
  if ((K & 7) || (K2 & 7) || (N & 7)) return ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(C) & 15) return ERR_BAD_ALIGN;
  if (epilogue == EPI_F32 ? (ldc & 3) : (ldc & 7)) return ERR_BAD_ALIGN;
  if (epilogue == EPI_BF16_RESID && (!R || (ldr & 7) || (reinterpret_cast<uintptr_t>(R) & 15)))
    return ERR_BAD_ALIGN;
  if (epilogue == EPI_SWIGLU && (!H || (ldh & 7) || (N & 31) || (reinterpret_cast<uintptr_t>(H) & 15)))
    return ERR_BAD_ALIGN;
  if (bn == 0) {
    // Largest tile that still yields at least ~one wave of CTAs.
    const long m_tiles = (M + GEMM_BM - 1) / GEMM_BM;
    const int sms = sm_count();
    if (N >= 256 && m_tiles * ((N + 255) / 256) >= sms) bn = 256;
    else if (N >= 128 && m_tiles * ((N + 127) / 128) >= sms / 2) bn = 128;
    else bn = (N > 64) ? 128 : 64;
  }
  if (bn != 64 && bn != 128 && bn != 256) return ERR_BAD_SHAPE;

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
                      reinterpret_cast<__nv_bfloat16*>(H), bias, ldc, ldr, ldh, M, N, epilogue}; \
    return launch_gemm<BN_, ST_>(tA, tB, tA2, tB2, kb_main, kb_extra, M, N, epi, status, max_ctas, \
                                 stream);                                                         \
  }
  if (bn == 256) ARTB_LAUNCH(256, 4)
  if (bn == 128) ARTB_LAUNCH(128, 6)
  ARTB_LAUNCH(64, 8)
#undef ARTB_LAUNCH
}
