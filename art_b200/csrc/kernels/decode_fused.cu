// Decode-time consumers of the split-K fp32 workspace.
//
// At decode batch sizes (M <= 512 rows) every projection is a weight-streaming split-K GEMM that accumulates
//     ws[:, 0:N)        = X W^T            (partial sums, fp32, vector atomics)
//     ws[:, N:N+kpad)   = X A_all^T        (the stacked LoRA shrink factors of all resident adapters as extra rows of W)
// Finishing such a product used to take three launches per projection (finalize + adapter-slot mask, LoRA expand GEMM,
// then the consumer: RMSNorm, or RoPE followed by the KV-cache write).  The two kernels here read the workspace once
// and do all of it, one CTA per token row:
//
//   decode_finalize_norm   y = ws + bias + residual + T_slot (sB_slot)^T ;  x_out = bf16(y) ;  h_out = RMSNorm(x_out) w
//                          (after the o and down projections; the norm is the next block's input norm)
//   decode_finalize_qkv    q|k|v = ws + bias + T_slot (sB_slot)^T ;  RoPE on q and k ;  q -> q_out, k / v -> KV cache
//
// A row belongs to ONE adapter slot, so the LoRA expand is a dot product of `cols` (= modules x rank, 8..24) shrink
// values with the row's slice of sB (kept transposed for this purpose, [shrink column, output feature]): CUDA-core
// work of a few MFLOP per layer, not worth a tensor-core launch.  Both kernels zero the workspace columns they
// consumed, which is what the next split-K GEMM expects.
//
// The reference gets these steps from vLLM's fused layers (src/art/local/vllm.py:22-84 patches that engine); the
// adapter-slot semantics are those of its punica SGMV path.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "bounds_check.cuh"
#include "host_utils.h"

namespace artb {

namespace {

struct alignas(16) bf8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  const bf8 r = *reinterpret_cast<const bf8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(r.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  bf8 r;
#pragma unroll
  for (int i = 0; i < 4; ++i) r.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf8*>(p) = r;
}

// reads 8 fp32 partial sums and leaves zeros behind
__device__ __forceinline__ void take8(float* w, float (&f)[8]) {
  float4* p = reinterpret_cast<float4*>(w);
  const float4 a = p[0], b = p[1];
  p[0] = make_float4(0.f, 0.f, 0.f, 0.f);
  p[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
}

// f[e] += sum_j t[j] * Bt[j * ldb + n0 + e],  j < cols; `Bt` (the scaled LoRA B, transposed: one row per shrink column,
// so that the threads of a warp read consecutive addresses) already points at the slot's first row.  The loads are
// issued eight at a time before any of them is used: one at a time, a row of `cols` dependent L2 round trips was the
// whole cost of these kernels.
__device__ __forceinline__ void lora_expand8(float (&f)[8], const float* t, const __nv_bfloat16* Bt, int ldb, int n0, int cols) {
  for (int j0 = 0; j0 < cols; j0 += 8) {
    bf8 b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (j0 + i < cols) b[i] = *reinterpret_cast<const bf8*>(Bt + static_cast<size_t>(j0 + i) * ldb + n0);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (j0 + i < cols) {
        const float tj = t[j0 + i];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 v = __bfloat1622float2(b[i].v[e]);
          f[2 * e] = fmaf(tj, v.x, f[2 * e]);
          f[2 * e + 1] = fmaf(tj, v.y, f[2 * e + 1]);
        }
      }
  }
}

// the same for two 8-element pieces of one row (the two halves of a RoPE pair): four rows, i.e. eight loads, at a time
__device__ __forceinline__ void lora_expand8x2(float (&f)[8], float (&g)[8], const float* t, const __nv_bfloat16* Bt, int ldb,
                                               int n0, int n1, int cols) {
  for (int j0 = 0; j0 < cols; j0 += 4) {
    bf8 b[4], c[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (j0 + i < cols) {
        const __nv_bfloat16* r = Bt + static_cast<size_t>(j0 + i) * ldb;
        b[i] = *reinterpret_cast<const bf8*>(r + n0);
        c[i] = *reinterpret_cast<const bf8*>(r + n1);
      }
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (j0 + i < cols) {
        const float tj = t[j0 + i];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 v = __bfloat1622float2(b[i].v[e]), w = __bfloat1622float2(c[i].v[e]);
          f[2 * e] = fmaf(tj, v.x, f[2 * e]);
          f[2 * e + 1] = fmaf(tj, v.y, f[2 * e + 1]);
          g[2 * e] = fmaf(tj, w.x, g[2 * e]);
          g[2 * e + 1] = fmaf(tj, w.y, g[2 * e + 1]);
        }
      }
  }
}

__device__ __forceinline__ void add_bias8(float (&f)[8], const float* bias) {
  const float4 a = *reinterpret_cast<const float4*>(bias), b = *reinterpret_cast<const float4*>(bias + 4);
  f[0] += a.x, f[1] += a.y, f[2] += a.z, f[3] += a.w, f[4] += b.x, f[5] += b.y, f[6] += b.z, f[7] += b.w;
}

// One CTA per token row.  512 threads: a 3584-wide row is one 8-element vector per thread, so the row costs a handful of
// dependent memory round trips instead of a loop of them (with 128 threads this kernel was slower than the three
// launches it replaces: ~7 warps per SM cannot hide the latency).
constexpr int DF_THREADS = 512;
constexpr int DF_MAX_COLS = 64;

// shrink values of the row's own slot -> shared memory; all kpad shrink columns of the workspace row -> 0
__device__ __forceinline__ int stage_shrink(float* wrow, int N, int kpad, int cols, const int* adapter, int row, float* t_s) {
  const int a = adapter ? adapter[row] : -1;
  if (a >= 0 && static_cast<int>(threadIdx.x) < cols) t_s[threadIdx.x] = wrow[N + a * cols + threadIdx.x];
  __syncthreads();
  if (adapter)
    for (int j = threadIdx.x * 4; j < kpad; j += blockDim.x * 4)
      *reinterpret_cast<float4*>(wrow + N + j) = make_float4(0.f, 0.f, 0.f, 0.f);
  return a;
}

}  // namespace

template <int MAX_VEC>
__global__ void __launch_bounds__(DF_THREADS, MAX_VEC == 1 ? 2 : 1)
decode_finalize_norm_kernel(float* __restrict__ ws, int ldw, int N, int kpad, const float* __restrict__ bias,
                            const __nv_bfloat16* __restrict__ R, int ldr, const int* __restrict__ adapter,
                            const __nv_bfloat16* __restrict__ B_all, int ldb, int cols,
                            const __nv_bfloat16* __restrict__ norm_w, float eps, __nv_bfloat16* __restrict__ x_out, int ldx,
                            __nv_bfloat16* __restrict__ h_out, int ldh) {
  __shared__ float t_s[DF_MAX_COLS];
  __shared__ float red[DF_THREADS / 32];
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  float* wrow = ws + static_cast<size_t>(row) * ldw;
  const int a = stage_shrink(wrow, N, kpad, cols, adapter, row, t_s);
  const int nvec = N >> 3;
  float vals[MAX_VEC][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    const int v = threadIdx.x + i * DF_THREADS;
    if (v < nvec) {
      const int n0 = v * 8;
      float f[8];
      take8(wrow + n0, f);
      if (bias) add_bias8(f, bias + n0);
      if (R) {
        float r[8];
        ld8(R + static_cast<size_t>(row) * ldr + n0, r);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += r[e];
      }
      if (a >= 0) lora_expand8(f, t_s, B_all + static_cast<size_t>(a) * cols * ldb, ldb, n0, cols);
      st8(x_out + static_cast<size_t>(row) * ldx + n0, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        // the norm sees the residual stream as it is stored: rounded to bf16
        vals[i][e] = __bfloat162float(__float2bfloat16(f[e]));
        ss += vals[i][e] * vals[i][e];
      }
    }
  }
  if (!norm_w) return;     // uniform for the whole grid
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < DF_THREADS / 32; ++i) tot += red[i];
  const float r = rsqrtf(tot / N + eps);
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    const int v = threadIdx.x + i * DF_THREADS;
    if (v < nvec) {
      float wv[8], o[8];
      ld8(norm_w + v * 8, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = __bfloat162float(__float2bfloat16(vals[i][e] * r)) * wv[e];
      st8(h_out + static_cast<size_t>(row) * ldh + v * 8, o);
    }
  }
}

// Columns of the workspace row: [ q: Hq heads | k: Hkv heads | v: Hkv heads | shrink: kpad ], heads of hd values.
// Rotate-half RoPE: the pair is (i, i + hd/2) inside a head, angle pos * theta^(-2i/hd).
// 256 threads, two CTAs per SM (128 registers each): the 320 (rope pair | v) units of a 7B row take two short passes
constexpr int DQ_THREADS = 256;

__global__ void __launch_bounds__(DQ_THREADS, 2)
decode_finalize_qkv_kernel(float* __restrict__ ws, int ldw, int Hq, int Hkv, int hd, int kpad,
                           const float* __restrict__ bias, const int* __restrict__ adapter,
                           const __nv_bfloat16* __restrict__ B_all, int ldb, int cols, const int* __restrict__ pos,
                           float log2_theta, const int* __restrict__ slot, __nv_bfloat16* __restrict__ k_cache,
                           __nv_bfloat16* __restrict__ v_cache, __nv_bfloat16* __restrict__ q_out, int ldq,
                           long num_slots, int* status) {
  __shared__ float t_s[DF_MAX_COLS];
  __shared__ float cs_s[128], sn_s[128];     // cos / sin of the row's position for every frequency: shared by all heads
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x;
  const int q_size = Hq * hd, kv_size = Hkv * hd, N = q_size + 2 * kv_size;
  float* wrow = ws + static_cast<size_t>(row) * ldw;
  if (static_cast<int>(threadIdx.x) < (hd >> 1)) {
    const float inv_freq = exp2f(-log2_theta * (2.f * threadIdx.x) / hd);
    sincosf(static_cast<float>(pos[row]) * inv_freq, &sn_s[threadIdx.x], &cs_s[threadIdx.x]);
  }
  const int a = stage_shrink(wrow, N, kpad, cols, adapter, row, t_s);      // contains the block barrier
  const __nv_bfloat16* Bs = B_all + (a >= 0 ? static_cast<size_t>(a) * cols * ldb : 0);
  int s = slot[row];
  if (s >= 0 && !index_ok(s, num_slots, status)) s = -1;      // checked build: a bad slot is reported, not written
  const int half = hd >> 1, per_head = half >> 3;
  const int rope_units = (Hq + Hkv) * per_head, v_units = kv_size >> 3;
  for (int u = threadIdx.x; u < rope_units + v_units; u += DQ_THREADS) {
    if (u < rope_units) {
      const int h = u / per_head, vv = u - h * per_head;
      const int c1 = h * hd + vv * 8, c2 = c1 + half;
      float x1[8], x2[8];
      take8(wrow + c1, x1);
      take8(wrow + c2, x2);
      if (bias) {
        add_bias8(x1, bias + c1);
        add_bias8(x2, bias + c2);
      }
      if (a >= 0) lora_expand8x2(x1, x2, t_s, Bs, ldb, c1, c2, cols);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float sn = sn_s[vv * 8 + e], cs = cs_s[vv * 8 + e];
        const float p = x1[e], q = x2[e];
        x1[e] = p * cs - q * sn;
        x2[e] = q * cs + p * sn;
      }
      if (h < Hq) {
        __nv_bfloat16* d = q_out + static_cast<size_t>(row) * ldq + c1;
        st8(d, x1);
        st8(d + half, x2);
      } else if (s >= 0) {
        __nv_bfloat16* d = k_cache + static_cast<size_t>(s) * kv_size + (c1 - q_size);
        st8(d, x1);
        st8(d + half, x2);
      }
    } else {
      const int c = q_size + kv_size + (u - rope_units) * 8;
      float x[8];
      take8(wrow + c, x);
      if (bias) add_bias8(x, bias + c);
      if (a >= 0) lora_expand8(x, t_s, Bs, ldb, c, cols);
      if (s >= 0) st8(v_cache + static_cast<size_t>(s) * kv_size + (c - q_size - kv_size), x);
    }
  }
}

}  // namespace artb

using namespace artb;

// ws fp32 [M, ldw]: columns [0, N) partial sums of the projection, [N, N + kpad) of the stacked LoRA shrink (only read
// when `adapter` is given: int32 [M], slot of the row or < 0).  B_all bf16 [kpad, ldb]: the scaled LoRA B of every slot,
// transposed (row = shrink column, `cols` rows per slot, <= 64; ldb >= N).  R: residual rows (optional).  norm_w null:
// no RMSNorm, h_out unused.
ARTB_EXPORT int artb_decode_finalize_norm(float* ws, int ldw, int M, int N, int kpad, const float* bias, const void* R,
                                          int ldr, const int* adapter, const void* B_all, int ldb, int cols,
                                          const void* norm_w, float eps, void* x_out, int ldx, void* h_out, int ldh,
                                          cudaStream_t st) {
  if (M <= 0) return 0;
  if ((N & 7) || (ldw & 3) || (ldx & 7) || (R && (ldr & 7)) || (norm_w && (!h_out || (ldh & 7)))) return ERR_BAD_SHAPE;
  if (adapter && (cols <= 0 || cols > DF_MAX_COLS || (kpad & 3) || (ldb & 7) || !B_all)) return ERR_BAD_SHAPE;
  if (N > DF_THREADS * 8 * 4) return ERR_TOO_LARGE;
  if ((reinterpret_cast<uintptr_t>(ws) & 15) || ((N * 4) & 15)) return ERR_BAD_ALIGN;
  const int per = (N / 8 + DF_THREADS - 1) / DF_THREADS;
#define ARTB_DF(V)                                                                                                      \
  return static_cast<int>(launch_kernel(                                                                                \
      decode_finalize_norm_kernel<V>, dim3(M), dim3(DF_THREADS), 0, st, ws, ldw, N, kpad, bias,                         \
      reinterpret_cast<const __nv_bfloat16*>(R), ldr, adapter, reinterpret_cast<const __nv_bfloat16*>(B_all), ldb, cols, \
      reinterpret_cast<const __nv_bfloat16*>(norm_w), eps, reinterpret_cast<__nv_bfloat16*>(x_out), ldx,                \
      reinterpret_cast<__nv_bfloat16*>(h_out), ldh))
  if (per <= 1) ARTB_DF(1);
  if (per <= 2) ARTB_DF(2);
  ARTB_DF(4);
#undef ARTB_DF
}

// k_cache / v_cache: [slots, Hkv * hd] bf16 (slot = block * block_size + offset; slot[m] < 0: row not written).
ARTB_EXPORT int artb_decode_finalize_qkv(float* ws, int ldw, int M, int Hq, int Hkv, int hd, int kpad, const float* bias,
                                         const int* adapter, const void* B_all, int ldb, int cols, const int* pos,
                                         float theta, const int* slot, void* k_cache, void* v_cache, void* q_out, int ldq,
                                         long num_slots, int* status, cudaStream_t st) {
  if (M <= 0) return 0;
  if ((hd & 15) || hd > 256 || (ldw & 3) || (ldq & 7) || Hq <= 0 || Hkv <= 0 || !pos || !slot) return ERR_BAD_SHAPE;
  if (adapter && (cols <= 0 || cols > DF_MAX_COLS || (kpad & 3) || (ldb & 7) || !B_all)) return ERR_BAD_SHAPE;
  if (reinterpret_cast<uintptr_t>(ws) & 15) return ERR_BAD_ALIGN;
  return static_cast<int>(launch_kernel(
      decode_finalize_qkv_kernel, dim3(M), dim3(DQ_THREADS), 0, st, ws, ldw, Hq, Hkv, hd, kpad, bias, adapter,
      reinterpret_cast<const __nv_bfloat16*>(B_all), ldb, cols, pos, log2f(theta), slot,
      reinterpret_cast<__nv_bfloat16*>(k_cache), reinterpret_cast<__nv_bfloat16*>(v_cache),
      reinterpret_cast<__nv_bfloat16*>(q_out), ldq, num_slots, status));
}

// Programmatic dependent launch for the kernels of the decode step (see pdl_switch in host_utils.h); returns the
// previous setting.  The engine turns it on around its decode body and off again afterwards.
ARTB_EXPORT int artb_set_pdl(int on) {
  const int prev = pdl_switch();
  pdl_switch() = on ? 1 : 0;
  return prev;
}
