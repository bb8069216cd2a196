// Tree-masked flash attention over packed rows, forward and backward, GQA.
//
// mask(q, k) = same packed row  AND  k <= q  AND  (group[q] == group[k] OR parent[q] == group[k])
//
// which lets a completion attend to itself and to the shared prompt it was sampled from,
// never to sibling completions (reference semantics: src/art/local/train.py:177-215, where
// the mask is a dense [B,S,S] bias handed to a generic attention backend).  Here the mask is
// evaluated from the two int32 id vectors inside the kernel, memory is O(S), and 64x64
// tiles that contain no allowed pair are skipped: a small prep kernel classifies every
// (q-block, k-block) tile once per micro-batch as empty / partial / full, and that table is
// reused by every layer's forward and backward.
//
// Forward: one CTA per (64-query block, q head, row); K/V tiles double-buffered with
// cp.async; QK^T and PV on warp-level tensor-core MMA (m16n8k16 bf16, fp32 accumulate);
// online softmax in the exp2 domain; writes O (bf16) and the log2-sum-exp per query.
// Backward: one CTA per (64-key block, kv head, row) looping over the q heads of the group
// and the q blocks at or after the key block; dK/dV stay in registers and are written once;
// dQ partials are accumulated into an fp32 buffer with atomics and converted afterwards.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "host_utils.h"

namespace artb {

constexpr int AT_B = 64;  // tile edge (queries and keys)

__device__ __forceinline__ void at_cp16(void* smem, const void* gmem) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void at_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void at_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ------------------------------------------------------------------ tile states
// state[(row * nb + qb) * nb + kb]: 0 = no allowed pair, 1 = some, 2 = all pairs allowed.
__global__ void attn_tile_state_kernel(const int* __restrict__ gid, const int* __restrict__ pid,
                                       uint8_t* __restrict__ state, int S, int nb) {
  const int qb = blockIdx.x, kb = blockIdx.y, row = blockIdx.z;
  uint8_t* out = state + (static_cast<size_t>(row) * nb + qb) * nb + kb;
  if (kb > qb) {
    if (threadIdx.x == 0) *out = 0;
    return;
  }
  __shared__ int gq[AT_B], pq[AT_B], gk[AT_B];
  const int base = row * S;
  if (threadIdx.x < AT_B) {
    gq[threadIdx.x] = gid[base + qb * AT_B + threadIdx.x];
    pq[threadIdx.x] = pid[base + qb * AT_B + threadIdx.x];
    gk[threadIdx.x] = gid[base + kb * AT_B + threadIdx.x];
  }
  __syncthreads();
  int any = 0, all = 1;
  for (int p = threadIdx.x; p < AT_B * AT_B; p += blockDim.x) {
    const int q = p / AT_B, k = p % AT_B;
    const bool ok = (kb * AT_B + k <= qb * AT_B + q) && (gk[k] == gq[q] || gk[k] == pq[q]);
    any |= ok;
    all &= ok;
  }
  any = __syncthreads_or(any);
  all = __syncthreads_and(all);
  if (threadIdx.x == 0) *out = any ? (all ? 2 : 1) : 0;
}

// ---------------------------------------------------------------------- forward
template <int HD>
__global__ void __launch_bounds__(128)
attn_tree_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, const int* __restrict__ gid,
                     const int* __restrict__ pid, const uint8_t* __restrict__ state,
                     __nv_bfloat16* __restrict__ out, int ldo, float* __restrict__ lse2, int S, int nb, int Hq,
                     int Hkv, float scale_log2, long M) {
  constexpr int LD = HD + 8;
  extern __shared__ __align__(16) uint8_t at_smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(at_smem);
  __nv_bfloat16* sK = sQ + AT_B * LD;          // [2][64][LD]
  __nv_bfloat16* sV = sK + 2 * AT_B * LD;      // [2][64][LD]
  int* sGk = reinterpret_cast<int*>(sV + 2 * AT_B * LD);  // [2][64]

  const int qb = nb - 1 - blockIdx.x;  // heavy (late) query blocks first
  const int h = blockIdx.y, row = blockIdx.z;
  const int kvh = h / (Hq / Hkv);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3, jm = lane >> 3, rr = lane & 7;
  const long base = static_cast<long>(row) * S;
  const uint8_t* st = state + (static_cast<size_t>(row) * nb + qb) * nb;

  const __nv_bfloat16* qptr = qkv + (base + qb * AT_B) * ld + h * HD;
  const __nv_bfloat16* kbase = qkv + base * ld + (Hq + kvh) * HD;
  const __nv_bfloat16* vbase = qkv + base * ld + (Hq + Hkv + kvh) * HD;

  constexpr int VEC_ROW = HD / 8;
  for (int v = tid; v < AT_B * VEC_ROW; v += 128) {
    const int r = v / VEC_ROW, c = v % VEC_ROW;
    at_cp16(sQ + r * LD + c * 8, qptr + static_cast<long>(r) * ld + c * 8);
  }
  at_commit();

  auto load_kv = [&](int kb, int stage) {
    const __nv_bfloat16* kp = kbase + static_cast<long>(kb) * AT_B * ld;
    const __nv_bfloat16* vp = vbase + static_cast<long>(kb) * AT_B * ld;
    for (int v = tid; v < AT_B * VEC_ROW; v += 128) {
      const int r = v / VEC_ROW, c = v % VEC_ROW;
      at_cp16(sK + (stage * AT_B + r) * LD + c * 8, kp + static_cast<long>(r) * ld + c * 8);
      at_cp16(sV + (stage * AT_B + r) * LD + c * 8, vp + static_cast<long>(r) * ld + c * 8);
    }
    if (tid < AT_B) sGk[stage * AT_B + tid] = gid[base + kb * AT_B + tid];
    at_commit();
  };
  auto next_valid = [&](int kb) {
    while (kb <= qb && st[kb] == 0) ++kb;
    return kb;
  };

  const int qrow0 = qb * AT_B + warp * 16 + g, qrow1 = qrow0 + 8;
  const int gq0 = gid[base + qrow0], pq0 = pid[base + qrow0];
  const int gq1 = gid[base + qrow1], pq1 = pid[base + qrow1];

  float acc_o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc_o[i][j] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  int kb = next_valid(0);
  int stage = 0;
  if (kb <= qb) load_kv(kb, 0);
  at_wait<0>();
  __syncthreads();
  // Q fragments stay in registers for the whole key loop
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks)
    ldsm_x4(qf[ks], sQ + (warp * 16 + (jm & 1) * 8 + rr) * LD + ks * 16 + (jm >> 1) * 8);

  while (kb <= qb) {
    const int kb_next = next_valid(kb + 1);
    if (kb_next <= qb) load_kv(kb_next, stage ^ 1);
    const __nv_bfloat16* cK = sK + stage * AT_B * LD;
    const __nv_bfloat16* cV = sV + stage * AT_B * LD;
    const int* cG = sGk + stage * AT_B;

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldsm_x4(b, cK + (np * 16 + (jm >> 1) * 8 + rr) * LD + ks * 16 + (jm & 1) * 8);
        mma16816(s[np * 2], qf[ks], b[0], b[1]);
        mma16816(s[np * 2 + 1], qf[ks], b[2], b[3]);
      }
    }
    const bool partial = st[kb] == 1;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int c = i * 8 + 2 * t + j;
        float x0 = s[i][j] * scale_log2, x1 = s[i][2 + j] * scale_log2;
        if (partial) {
          const int kidx = kb * AT_B + c;
          const int gk = cG[c];
          if (!(kidx <= qrow0 && (gk == gq0 || gk == pq0))) x0 = -INFINITY;
          if (!(kidx <= qrow1 && (gk == gq1 || gk == pq1))) x1 = -INFINITY;
        }
        s[i][j] = x0;
        s[i][2 + j] = x1;
        mx0 = fmaxf(mx0, x0);
        mx1 = fmaxf(mx1, x1);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
    const float c0 = exp2f(m0 - ms0), c1 = exp2f(m1 - ms1);
    m0 = mn0;
    m1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
    uint32_t pf[4][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float p00 = exp2f(s[i][0] - ms0), p01 = exp2f(s[i][1] - ms0);
      const float p10 = exp2f(s[i][2] - ms1), p11 = exp2f(s[i][3] - ms1);
      rs0 += p00 + p01;
      rs1 += p10 + p11;
      pf[i >> 1][(i & 1) * 2] = pack2(p00, p01);
      pf[i >> 1][(i & 1) * 2 + 1] = pack2(p10, p11);
    }
    l0 = l0 * c0 + rs0;
    l1 = l1 * c1 + rs1;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      acc_o[i][0] *= c0;
      acc_o[i][1] *= c0;
      acc_o[i][2] *= c1;
      acc_o[i][3] *= c1;
    }
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t b[4];
        ldsm_x4_t(b, cV + (ks * 16 + (jm & 1) * 8 + rr) * LD + dp * 16 + (jm >> 1) * 8);
        mma16816(acc_o[dp * 2], pf[ks], b[0], b[1]);
        mma16816(acc_o[dp * 2 + 1], pf[ks], b[2], b[3]);
      }
    }
    at_wait<0>();
    __syncthreads();
    kb = kb_next;
    stage ^= 1;
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  __nv_bfloat16* o0 = out + (base + qrow0) * ldo + h * HD;
  __nv_bfloat16* o1 = out + (base + qrow1) * ldo + h * HD;
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    *reinterpret_cast<uint32_t*>(o0 + i * 8 + 2 * t) = pack2(acc_o[i][0] * inv0, acc_o[i][1] * inv0);
    *reinterpret_cast<uint32_t*>(o1 + i * 8 + 2 * t) = pack2(acc_o[i][2] * inv1, acc_o[i][3] * inv1);
  }
  if (t == 0) {
    lse2[static_cast<long>(h) * M + base + qrow0] = m0 + log2f(l0);
    lse2[static_cast<long>(h) * M + base + qrow1] = m1 + log2f(l1);
  }
}

// ------------------------------------------------------------ D = rowsum(dO * O)
__global__ void attn_dot_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O, int ld,
                                float* __restrict__ D, long M, int Hq, int HD) {
  const long wid = blockIdx.x * static_cast<long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= M * Hq) return;
  const long m = wid / Hq;
  const int h = wid % Hq;
  const __nv_bfloat16* a = dO + m * ld + h * HD;
  const __nv_bfloat16* b = O + m * ld + h * HD;
  float s = 0.f;
  for (int i = lane * 2; i < HD; i += 64) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + i));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + i));
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) D[static_cast<long>(h) * M + m] = s;
}

// --------------------------------------------------------------------- backward
template <int HD>
__global__ void __launch_bounds__(128)
attn_tree_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, const __nv_bfloat16* __restrict__ dO, int ldo,
                     const int* __restrict__ gid, const int* __restrict__ pid, const uint8_t* __restrict__ state,
                     const float* __restrict__ lse2, const float* __restrict__ Dv, float* __restrict__ dq_acc,
                     __nv_bfloat16* __restrict__ dqkv, int S, int nb, int Hq, int Hkv, float scale,
                     float scale_log2, long M) {
  constexpr int LD = HD + 8;
  constexpr int SLD = AT_B + 8;
  constexpr int TILE = AT_B * LD;
  extern __shared__ __align__(16) uint8_t at_smem[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(at_smem);
  __nv_bfloat16* sV = sK + TILE;
  __nv_bfloat16* sQ = sV + TILE;        // [2][TILE]  double-buffered
  __nv_bfloat16* sdO = sQ + 2 * TILE;   // [2][TILE]
  __nv_bfloat16* sdS = sdO + 2 * TILE;  // [key][query]
  float* sL = reinterpret_cast<float*>(sdS + AT_B * SLD);  // [2][64]
  float* sD = sL + 2 * AT_B;
  int* sGq = reinterpret_cast<int*>(sD + 2 * AT_B);
  int* sPq = sGq + 2 * AT_B;

  const int kb = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
  const int G = Hq / Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3, jm = lane >> 3, rr = lane & 7;
  const long base = static_cast<long>(row) * S;
  constexpr int VEC_ROW = HD / 8;
  const uint8_t* st_col = state + static_cast<size_t>(row) * nb * nb + kb;  // + qb * nb

  const __nv_bfloat16* kptr = qkv + (base + kb * AT_B) * ld + (Hq + kvh) * HD;
  const __nv_bfloat16* vptr = qkv + (base + kb * AT_B) * ld + (Hq + Hkv + kvh) * HD;
  for (int v = tid; v < AT_B * VEC_ROW; v += 128) {
    const int r = v / VEC_ROW, c = v % VEC_ROW;
    at_cp16(sK + r * LD + c * 8, kptr + static_cast<long>(r) * ld + c * 8);
    at_cp16(sV + r * LD + c * 8, vptr + static_cast<long>(r) * ld + c * 8);
  }

  // work list: (hq, qb) pairs with a non-empty tile, visited in order; item index -> (hq, qb)
  const int nq = nb - kb;
  const int n_items = G * nq;
  auto next_item = [&](int it) {
    while (it < n_items && st_col[static_cast<size_t>(kb + it % nq) * nb] == 0) ++it;
    return it;
  };
  auto load_item = [&](int it, int buf) {
    const int hq = kvh * G + it / nq, qb = kb + it % nq;
    const __nv_bfloat16* qptr = qkv + (base + qb * AT_B) * ld + hq * HD;
    const __nv_bfloat16* doptr = dO + (base + qb * AT_B) * ldo + hq * HD;
    for (int v = tid; v < AT_B * VEC_ROW; v += 128) {
      const int r = v / VEC_ROW, c = v % VEC_ROW;
      at_cp16(sQ + buf * TILE + r * LD + c * 8, qptr + static_cast<long>(r) * ld + c * 8);
      at_cp16(sdO + buf * TILE + r * LD + c * 8, doptr + static_cast<long>(r) * ldo + c * 8);
    }
    if (tid < AT_B) {
      const long qi = base + qb * AT_B + tid;
      sL[buf * AT_B + tid] = lse2[static_cast<long>(hq) * M + qi];
      sD[buf * AT_B + tid] = Dv[static_cast<long>(hq) * M + qi];
      sGq[buf * AT_B + tid] = gid[qi];
      sPq[buf * AT_B + tid] = pid[qi];
    }
    at_commit();
  };

  const int krow0 = kb * AT_B + warp * 16 + g, krow1 = krow0 + 8;
  const int gk0 = gid[base + krow0], gk1 = gid[base + krow1];

  float dk[HD / 8][4], dv[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) dk[i][j] = dv[i][j] = 0.f;

  int it = next_item(0);
  int buf = 0;
  if (it < n_items) load_item(it, 0);   // same async group as K/V
  else at_commit();
  while (it < n_items) {
    const int it_next = next_item(it + 1);
    if (it_next < n_items) {
      load_item(it_next, buf ^ 1);      // buffer buf^1 was released by the barrier that ended the last iteration
      at_wait<1>();
    } else {
      at_wait<0>();
    }
    __syncthreads();
    const int hq = kvh * G + it / nq, qb = kb + it % nq;
    const uint8_t stt = st_col[static_cast<size_t>(qb) * nb];
    const __nv_bfloat16* cQ = sQ + buf * TILE;
    const __nv_bfloat16* cdO = sdO + buf * TILE;
    const float* cL = sL + buf * AT_B;
    const float* cD = sD + buf * AT_B;
    const int* cGq = sGq + buf * AT_B;
    const int* cPq = sPq + buf * AT_B;

    // S^T = K_w Q^T  and  dP^T = V_w dO^T   (16 keys x 64 queries per warp)
    float sT[8][4], dpT[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) sT[i][j] = dpT[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t ka[4], va[4];
      ldsm_x4(ka, sK + (warp * 16 + (jm & 1) * 8 + rr) * LD + ks * 16 + (jm >> 1) * 8);
      ldsm_x4(va, sV + (warp * 16 + (jm & 1) * 8 + rr) * LD + ks * 16 + (jm >> 1) * 8);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldsm_x4(b, cQ + (np * 16 + (jm >> 1) * 8 + rr) * LD + ks * 16 + (jm & 1) * 8);
        mma16816(sT[np * 2], ka, b[0], b[1]);
        mma16816(sT[np * 2 + 1], ka, b[2], b[3]);
        ldsm_x4(b, cdO + (np * 16 + (jm >> 1) * 8 + rr) * LD + ks * 16 + (jm & 1) * 8);
        mma16816(dpT[np * 2], va, b[0], b[1]);
        mma16816(dpT[np * 2 + 1], va, b[2], b[3]);
      }
    }
    // P^T and dS^T (rows: keys g / g+8 of this warp; cols: queries)
    uint32_t pA[4][4], dsA[4][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float p[4], ds[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = i * 8 + 2 * t + (j & 1);      // query index within the tile
        const int kr = (j < 2) ? krow0 : krow1;
        const int gk = (j < 2) ? gk0 : gk1;
        bool ok = true;
        if (stt == 1) ok = (kr <= qb * AT_B + c) && (gk == cGq[c] || gk == cPq[c]);
        const float pv = ok ? exp2f(sT[i][j] * scale_log2 - cL[c]) : 0.f;
        p[j] = pv;
        ds[j] = pv * (dpT[i][j] - cD[c]) * scale;
      }
      pA[i >> 1][(i & 1) * 2] = pack2(p[0], p[1]);
      pA[i >> 1][(i & 1) * 2 + 1] = pack2(p[2], p[3]);
      dsA[i >> 1][(i & 1) * 2] = pack2(ds[0], ds[1]);
      dsA[i >> 1][(i & 1) * 2 + 1] = pack2(ds[2], ds[3]);
      // stash dS^T for the dQ product: sdS[key][query]
      *reinterpret_cast<uint32_t*>(sdS + (warp * 16 + g) * SLD + i * 8 + 2 * t) = pack2(ds[0], ds[1]);
      *reinterpret_cast<uint32_t*>(sdS + (warp * 16 + g + 8) * SLD + i * 8 + 2 * t) = pack2(ds[2], ds[3]);
    }
    // dV_w += P^T dO ;  dK_w += dS^T Q     (contraction over the 64 queries)
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t b[4];
        ldsm_x4_t(b, cdO + (ks * 16 + (jm & 1) * 8 + rr) * LD + dp * 16 + (jm >> 1) * 8);
        mma16816(dv[dp * 2], pA[ks], b[0], b[1]);
        mma16816(dv[dp * 2 + 1], pA[ks], b[2], b[3]);
        ldsm_x4_t(b, cQ + (ks * 16 + (jm & 1) * 8 + rr) * LD + dp * 16 + (jm >> 1) * 8);
        mma16816(dk[dp * 2], dsA[ks], b[0], b[1]);
        mma16816(dk[dp * 2 + 1], dsA[ks], b[2], b[3]);
      }
    }
    __syncthreads();  // sdS complete
    // dQ_w[16 queries x HD] = dS[16 q x 64 keys] K[64 keys x HD], in two halves of HD
    float* dq0 = dq_acc + (base + qb * AT_B + warp * 16 + g) * (static_cast<long>(Hq) * HD) + hq * HD;
    float* dq1 = dq0 + 8L * Hq * HD;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      float dq[HD / 16][4];
#pragma unroll
      for (int i = 0; i < HD / 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) dq[i][j] = 0.f;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t a[4];
        // A = dS (rows: queries, k: keys) read transposed from sdS[key][query]
        ldsm_x4_t(a, sdS + (ks * 16 + (jm >> 1) * 8 + rr) * SLD + warp * 16 + (jm & 1) * 8);
#pragma unroll
        for (int dp = 0; dp < HD / 32; ++dp) {
          uint32_t b[4];
          ldsm_x4_t(b, sK + (ks * 16 + (jm & 1) * 8 + rr) * LD + half * (HD / 2) + dp * 16 + (jm >> 1) * 8);
          mma16816(dq[dp * 2], a, b[0], b[1]);
          mma16816(dq[dp * 2 + 1], a, b[2], b[3]);
        }
      }
#pragma unroll
      for (int i = 0; i < HD / 16; ++i) {
        const int col = half * (HD / 2) + i * 8 + 2 * t;
        atomicAdd(reinterpret_cast<float2*>(dq0 + col), make_float2(dq[i][0], dq[i][1]));
        atomicAdd(reinterpret_cast<float2*>(dq1 + col), make_float2(dq[i][2], dq[i][3]));
      }
    }
    __syncthreads();  // all reads of this iteration's buffers and of sdS are done
    it = it_next;
    buf ^= 1;
  }
  at_wait<0>();
  // write dK, dV (bf16) into the fused gradient buffer
  __nv_bfloat16* dk0 = dqkv + (base + krow0) * ld + (Hq + kvh) * HD;
  __nv_bfloat16* dk1 = dqkv + (base + krow1) * ld + (Hq + kvh) * HD;
  __nv_bfloat16* dv0 = dqkv + (base + krow0) * ld + (Hq + Hkv + kvh) * HD;
  __nv_bfloat16* dv1 = dqkv + (base + krow1) * ld + (Hq + Hkv + kvh) * HD;
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    *reinterpret_cast<uint32_t*>(dk0 + i * 8 + 2 * t) = pack2(dk[i][0], dk[i][1]);
    *reinterpret_cast<uint32_t*>(dk1 + i * 8 + 2 * t) = pack2(dk[i][2], dk[i][3]);
    *reinterpret_cast<uint32_t*>(dv0 + i * 8 + 2 * t) = pack2(dv[i][0], dv[i][1]);
    *reinterpret_cast<uint32_t*>(dv1 + i * 8 + 2 * t) = pack2(dv[i][2], dv[i][3]);
  }
}

// fp32 dQ accumulator [M, Hq*HD] -> bf16 into the q columns of dqkv [M, ld]
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dqkv, int ld,
                                       long M, int QW) {
  const int vec = QW >> 2;
  const long total = M * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long m = i / vec;
    const int c = (i % vec) * 4;
    const float4 v = *reinterpret_cast<const float4*>(acc + m * QW + c);
    uint2 o;
    o.x = pack2(v.x, v.y);
    o.y = pack2(v.z, v.w);
    *reinterpret_cast<uint2*>(dqkv + m * ld + c) = o;
  }
}

template <int HD>
static int fwd_smem() { return (AT_B * (HD + 8) * 5) * 2 + 2 * AT_B * 4; }
template <int HD>
static int bwd_smem() { return (AT_B * (HD + 8) * 6 + AT_B * (AT_B + 8)) * 2 + 8 * AT_B * 4; }

}  // namespace artb

using namespace artb;
typedef __nv_bfloat16 bf16;

// state: uint8 [rows, nb, nb] with nb = S / 64.
ARTB_EXPORT int artb_attn_tile_states(const int* gid, const int* pid, uint8_t* state, int rows, int S,
                                      cudaStream_t st) {
  if (S % AT_B) return ERR_BAD_SHAPE;
  const int nb = S / AT_B;
  dim3 grid(nb, nb, rows);
  attn_tile_state_kernel<<<grid, 256, 0, st>>>(gid, pid, state, S, nb);
  return (int)cudaGetLastError();
}

// qkv [rows*S, ld] post-RoPE (q | k | v columns); out [rows*S, Hq*hd]; lse2 [Hq, rows*S] (log2 domain).
ARTB_EXPORT int artb_attn_tree_fwd(const void* qkv, int ld, const int* gid, const int* pid, const uint8_t* state,
                                   void* out, int ldo, float* lse2, int rows, int S, int Hq, int Hkv, int hd,
                                   cudaStream_t st) {
  if (S % AT_B || Hq % Hkv || (ld & 7) || (ldo & 7)) return ERR_BAD_SHAPE;
  const int nb = S / AT_B;
  const long M = (long)rows * S;
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  dim3 grid(nb, Hq, rows);
#define ARTB_FWD(HD_)                                                                                           \
  {                                                                                                             \
    static bool cfgd = false;                                                                                   \
    if (!cfgd) {                                                                                                \
      cudaFuncSetAttribute(attn_tree_fwd_kernel<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<HD_>()); \
      cfgd = true;                                                                                              \
    }                                                                                                           \
    attn_tree_fwd_kernel<HD_><<<grid, 128, fwd_smem<HD_>(), st>>>((const bf16*)qkv, ld, gid, pid, state, (bf16*)out, \
                                                                  ldo, lse2, S, nb, Hq, Hkv, scale_log2, M);    \
  }
  if (hd == 128) ARTB_FWD(128)
  else if (hd == 64) ARTB_FWD(64)
  else if (hd == 32) ARTB_FWD(32)
  else return ERR_BAD_SHAPE;
#undef ARTB_FWD
  return (int)cudaGetLastError();
}

// dqkv [rows*S, ld] receives dq | dk | dv; dq_acc fp32 [rows*S, Hq*hd] scratch (zeroed here); Dbuf fp32 [Hq, rows*S].
ARTB_EXPORT int artb_attn_tree_bwd(const void* qkv, int ld, const void* out, const void* dout, int ldo,
                                   const int* gid, const int* pid, const uint8_t* state, const float* lse2,
                                   float* Dbuf, float* dq_acc, void* dqkv, int rows, int S, int Hq, int Hkv, int hd,
                                   cudaStream_t st) {
  if (S % AT_B || Hq % Hkv || (ld & 7) || (ldo & 7)) return ERR_BAD_SHAPE;
  const int nb = S / AT_B;
  const long M = (long)rows * S;
  const float scale = 1.f / sqrtf((float)hd);
  const float scale_log2 = 1.4426950408889634f * scale;
  cudaMemsetAsync(dq_acc, 0, sizeof(float) * M * Hq * hd, st);
  {
    const long warps = M * Hq;
    attn_dot_kernel<<<(unsigned)((warps + 3) / 4), 128, 0, st>>>((const bf16*)dout, (const bf16*)out, ldo, Dbuf, M, Hq, hd);
  }
  dim3 grid(nb, Hkv, rows);
#define ARTB_BWD(HD_)                                                                                           \
  {                                                                                                             \
    static bool cfgd = false;                                                                                   \
    if (!cfgd) {                                                                                                \
      cudaFuncSetAttribute(attn_tree_bwd_kernel<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd_smem<HD_>()); \
      cfgd = true;                                                                                              \
    }                                                                                                           \
    attn_tree_bwd_kernel<HD_><<<grid, 128, bwd_smem<HD_>(), st>>>((const bf16*)qkv, ld, (const bf16*)dout, ldo, gid, \
                                                                  pid, state, lse2, Dbuf, dq_acc, (bf16*)dqkv, S, \
                                                                  nb, Hq, Hkv, scale, scale_log2, M);           \
  }
  if (hd == 128) ARTB_BWD(128)
  else if (hd == 64) ARTB_BWD(64)
  else if (hd == 32) ARTB_BWD(32)
  else return ERR_BAD_SHAPE;
#undef ARTB_BWD
  {
    const int QW = Hq * hd;
    long total = M * (QW / 4);
    long blocks = (total + 255) / 256;
    if (blocks > 148L * 16) blocks = 148L * 16;
    attn_dq_convert_kernel<<<(unsigned)blocks, 256, 0, st>>>(dq_acc, (bf16*)dqkv, ld, M, QW);
  }
  return (int)cudaGetLastError();
}
