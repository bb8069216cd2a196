// LoRA factor gradients: OUT[C, R] += P[M, C]^T * Q[M, R]   (bf16 in, fp32 accumulate)
//
// Both LoRA weight gradients are contractions over the token dimension between one wide
// activation matrix and one skinny one:
//     dB_cat[N, R]   += dY[M, N]^T * T[M, R]          (T = X A^T, saved by the forward)
//     dA_cat^T[K, R] += X[M, K]^T  * dT[M, R]         (dT = dY (sB))
// R is the padded LoRA width (64).  The op reads the wide matrix exactly once and does
// R/8 times fewer FLOPs than a square GEMM, so it is bandwidth-bound; warp-level
// mma.sync (m16n8k16) with ldmatrix.trans from padded shared tiles is enough to keep up
// with HBM.  Token-dimension splits accumulate with fp32 atomics.
//
// Counterpart in the reference: autograd through the PEFT/Unsloth LoRA modules
// (src/art/local/state.py:86-92, backward driven from src/art/local/train.py via HF Trainer).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_utils.h"

namespace artb {

constexpr int WG_BC = 128;   // columns of P per CTA
constexpr int WG_R = 64;     // columns of Q
constexpr int WG_BM = 32;    // token rows per pipeline chunk
constexpr int WG_PLD = WG_BC + 8;
constexpr int WG_QLD = WG_R + 8;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128)
lora_wgrad_kernel(const __nv_bfloat16* __restrict__ P, int ldp, const __nv_bfloat16* __restrict__ Q, int ldq,
                  float* __restrict__ out, int ldo, int M, int C, int rows_per_split,
                  const int* __restrict__ seg_off, long out_stride) {
  __shared__ __align__(16) __nv_bfloat16 sP[2][WG_BM][WG_PLD];
  __shared__ __align__(16) __nv_bfloat16 sQ[2][WG_BM][WG_QLD];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c0 = blockIdx.x * WG_BC;
  int m_begin = blockIdx.y * rows_per_split;
  int m_end = min(M, m_begin + rows_per_split);
  if (seg_off) {
    // grouped: blockIdx.z is the expert; its row segment is split evenly over gridDim.y CTAs
    // (clipped to the M rows the operands really have, whatever the offsets say)
    const int lo = min(seg_off[blockIdx.z], M), hi = min(seg_off[blockIdx.z + 1], M);
    const int rows = ((hi - lo + static_cast<int>(gridDim.y) - 1) / static_cast<int>(gridDim.y) + WG_BM - 1) / WG_BM * WG_BM;
    m_begin = lo + blockIdx.y * rows;
    m_end = min(hi, m_begin + rows);
    out += blockIdx.z * out_stride;
  }
  if (m_begin >= m_end) return;
  const int chunks = (m_end - m_begin + WG_BM - 1) / WG_BM;

  auto load_chunk = [&](int chunk, int stage) {
    const int m0 = m_begin + chunk * WG_BM;
#pragma unroll
    for (int i = 0; i < 4; ++i) {  // P: 32 rows x 16 vec
      const int v = tid + i * 128;
      const int r = v >> 4, cv = v & 15;
      const int gm = m0 + r, gc = c0 + cv * 8;
      const bool ok = gm < m_end && gc < C;
      cp_async16(&sP[stage][r][cv * 8], P + (ok ? static_cast<size_t>(gm) * ldp + gc : 0), ok);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {  // Q: 32 rows x 8 vec
      const int v = tid + i * 128;
      const int r = v >> 3, cv = v & 7;
      const int gm = m0 + r;
      const bool ok = gm < m_end;
      cp_async16(&sQ[stage][r][cv * 8], Q + (ok ? static_cast<size_t>(gm) * ldq + cv * 8 : 0), ok);
    }
    cp_async_commit();
  };

  float acc[2][8][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int k = 0; k < 4; ++k) acc[i][j][k] = 0.f;

  load_chunk(0, 0);
  for (int ch = 0; ch < chunks; ++ch) {
    const int st = ch & 1;
    if (ch + 1 < chunks) {
      load_chunk(ch + 1, st ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int j = lane >> 3, rr = lane & 7;  // ldmatrix: lane supplies row rr of matrix j
#pragma unroll
    for (int ks = 0; ks < WG_BM / 16; ++ks) {
      const int k0 = ks * 16;
      uint32_t a[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) {
        // A = P^T tile: rows = columns c of P, k = token.  smem is [k][c] -> transposed load.
        const int cbase = warp * 32 + mi * 16;
        const int krow = k0 + (j >> 1) * 8 + rr;
        const int ccol = cbase + (j & 1) * 8;
        ldmatrix_x4_trans(a[mi], &sP[st][krow][ccol]);
      }
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        // B = Q tile [k][n] -> transposed load gives the col-major fragments of two n8 blocks.
        uint32_t b[4];
        const int krow = k0 + (j & 1) * 8 + rr;
        const int ncol = nb * 16 + (j >> 1) * 8;
        ldmatrix_x4_trans(b, &sQ[st][krow][ncol]);
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
          mma_bf16(acc[mi][nb * 2], a[mi], b[0], b[1]);
          mma_bf16(acc[mi][nb * 2 + 1], a[mi], b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
    for (int nj = 0; nj < 8; ++nj) {
      const int col = nj * 8 + 2 * t;
      const int r0 = c0 + warp * 32 + mi * 16 + g;
      if (r0 < C) {
        atomicAdd(out + static_cast<size_t>(r0) * ldo + col, acc[mi][nj][0]);
        atomicAdd(out + static_cast<size_t>(r0) * ldo + col + 1, acc[mi][nj][1]);
      }
      if (r0 + 8 < C) {
        atomicAdd(out + static_cast<size_t>(r0 + 8) * ldo + col, acc[mi][nj][2]);
        atomicAdd(out + static_cast<size_t>(r0 + 8) * ldo + col + 1, acc[mi][nj][3]);
      }
    }
  }
}

}  // namespace artb

using namespace artb;

// out[C, 64] (fp32, ld = ldo) += P[M, C]^T Q[M, 64].  C % 8 == 0; P, Q 16-byte aligned rows.
ARTB_EXPORT int artb_lora_wgrad(const void* P, int ldp, const void* Q, int ldq, float* out, int ldo, int M, int C,
                                cudaStream_t st) {
  if (M <= 0 || C <= 0) return 0;
  if ((C & 7) || (ldp & 7) || (ldq & 7) || ldo < WG_R) return ERR_BAD_SHAPE;
  const int cblocks = (C + WG_BC - 1) / WG_BC;
  int splits = (4 * sm_count() + cblocks - 1) / cblocks;
  const int max_splits = (M + 4 * WG_BM - 1) / (4 * WG_BM);
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  int rows = (M + splits - 1) / splits;
  rows = (rows + WG_BM - 1) / WG_BM * WG_BM;
  splits = (M + rows - 1) / rows;
  dim3 grid(cblocks, splits);
  lora_wgrad_kernel<<<grid, 128, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(P), ldp,
                                          reinterpret_cast<const __nv_bfloat16*>(Q), ldq, out, ldo, M, C, rows,
                                          nullptr, 0);
  return static_cast<int>(cudaGetLastError());
}


// Grouped form for expert-sorted rows: out[e][C, 64] += P[seg_e, C]^T Q[seg_e, 64] for every expert e,
// seg_e = rows seg_off[e] .. seg_off[e+1] (device array, padded rows are zero).  One launch covers all experts.
ARTB_EXPORT int artb_lora_wgrad_grouped(const void* P, int ldp, const void* Q, int ldq, float* out, int ldo,
                                        long out_stride, const int* seg_off, int num_experts, int C, int splits,
                                        int rows, cudaStream_t st) {
  if (num_experts <= 0 || C <= 0 || rows <= 0) return 0;
  if ((C & 7) || (ldp & 7) || (ldq & 7) || ldo < WG_R || splits < 1) return ERR_BAD_SHAPE;
  dim3 grid((C + WG_BC - 1) / WG_BC, splits, num_experts);
  lora_wgrad_kernel<<<grid, 128, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(P), ldp,
                                          reinterpret_cast<const __nv_bfloat16*>(Q), ldq, out, ldo, rows, C, 0, seg_off,
                                          out_stride);
  return static_cast<int>(cudaGetLastError());
}
