// Tree-masked flash attention forward on tcgen05 / TMEM (head dim 128).
//
// One CTA = one 128-query tile of one head.  Warp roles: warp 0 issues TMA loads (Q once, then a
// 2-stage ring of K and V^T tiles), warp 1 issues tcgen05.mma, warps 2-5 (one thread per query
// row = one TMEM lane) run the online softmax and own the output accumulator.
//
//   S  = Q K^T          UMMA 128 x 128 x 128, A = Q tile, B = K tile (both K-major along the head dim)
//   P  = exp2(S*c - m)  softmax warps: TMEM -> registers (one read; the half row stays in registers),
//                       mask from group / parent ids on partially masked tiles only, bf16 P written
//                       to shared memory in the 128-byte-swizzled K-major layout UMMA reads
//   PV = P V            UMMA 128 x 128 x 128, A = P (shared memory), B = V^T tile (K-major along keys;
//                       V^T is a pre-transposed copy, 8 MB per layer, so that no operand needs an
//                       MN-major descriptor)
//   O  = O * 2^(m_old - m_new) + PV   in registers, one tile behind the softmax so that the tensor
//                       core works on S of tile j+1 and PV of tile j while the warps exponentiate
//
// TMEM: two S buffers and two PV buffers of 128 fp32 columns = 512 columns.  Fully masked 128 x 128
// tiles are skipped from the 64 x 64 tile-state table of the mma.sync kernels (attn_tree.cu); the log-sum-exp
// convention (log2 domain, scale folded in) is the same, so the existing backward kernel consumes this
// forward's output.  Every wait is bounded; on expiry the CTA records a status code and unwinds.
//
// Reference semantics: src/art/local/train.py:177-215 (dense additive bias) + SDPA.
#include <cuda_bf16.h>

#include "host_utils.h"
#include "ptx_sm100.cuh"

namespace artb {

constexpr int TC_B = 128;                 // queries per CTA, keys per tile
constexpr int TC_HD = 128;
constexpr int TC_TILE = TC_B * TC_HD * 2; // 32 KB: two 16 KB halves of 64 columns (one swizzle atom wide)
constexpr int TC_HALF = TC_TILE / 2;
constexpr int TC_THREADS = 320;           // TMA warp, MMA warp, 8 softmax warps

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct TcSmem {
  static constexpr int Q = 0;
  static constexpr int K = Q + TC_TILE;            // [2]
  static constexpr int V = K + 2 * TC_TILE;        // [2]
  static constexpr int P = V + 2 * TC_TILE;
  static constexpr int GK = P + TC_TILE;           // int [8 warps][64]: key group ids of a partially masked tile
  static constexpr int XCH = GK + 8 * 64 * 4;      // float [2][2][128]: row max / row sum exchange between warp pairs
  static constexpr int BAR = XCH + 2 * 256 * 4;    // 21 mbarriers + tmem slot + abort
  static constexpr int TOTAL = BAR + 28 * 8 + 1024;
};

// k-step kk (16 elements) of a [128 x 128] K-major tile stored as two 64-column halves
__device__ __forceinline__ uint64_t tc_desc(uint32_t tile_base, int kk) {
  return umma_smem_desc_k128(tile_base + (kk >> 2) * TC_HALF) + 2 * (kk & 3);
}

__device__ __forceinline__ int tc_state128(const uint8_t* st64, int nb64, int qb, int kb) {
  const uint8_t* r0 = st64 + static_cast<size_t>(2 * qb) * nb64 + 2 * kb;
  const uint8_t* r1 = r0 + nb64;
  const int a = r0[0], b = r0[1], c = r1[0], d = r1[1];
  if ((a | b | c | d) == 0) return 0;
  return (a == 2 && b == 2 && c == 2 && d == 2) ? 2 : 1;
}

__global__ void __launch_bounds__(TC_THREADS, 1)
attn_tc_fwd_kernel(const __grid_constant__ CUtensorMap tmQK, const __grid_constant__ CUtensorMap tmVt,
                   const int* __restrict__ gid, const int* __restrict__ pid, const uint8_t* __restrict__ state,
                   __nv_bfloat16* __restrict__ out, int ldo, float* __restrict__ lse2, int S, int Hq, int Hkv,
                   float scale_log2, long M, int* status) {
  extern __shared__ uint8_t tc_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TcSmem::BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* v_full = bars + 3;      // [2]
  uint64_t* kv_empty = bars + 5;    // [2]
  uint64_t* s_full = bars + 7;      // [2]
  uint64_t* s_empty = bars + 9;     // [2]
  uint64_t* p_full = bars + 11;
  uint64_t* p_empty = bars + 12;
  uint64_t* pv_full = bars + 13;    // [2]
  uint64_t* pv_empty = bars + 15;   // [2]
  uint64_t* x_bar = bars + 17;      // [4] one per lane quarter, two arrivals (the warp pair)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* sGk = reinterpret_cast<int*>(smem + TcSmem::GK);
  float* xch = reinterpret_cast<float*>(smem + TcSmem::XCH);

  const int nb = S / TC_B, nb64 = S / 64;
  const int qb = nb - 1 - blockIdx.x;      // heavy (late) query tiles first
  const int h = blockIdx.y, row = blockIdx.z;
  const int kvh = h / (Hq / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long base = static_cast<long>(row) * S;
  const uint8_t* st64 = state + static_cast<size_t>(row) * nb64 * nb64;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 8);
      mbar_init(&pv_full[i], 1);
      mbar_init(&pv_empty[i], 8);
    }
    for (int i = 0; i < 4; ++i) mbar_init(&x_bar[i], 2);
    mbar_init(p_full, 8);
    mbar_init(p_empty, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmQK);
      tma_prefetch_desc(&tmVt);
      mbar_expect_tx(q_full, TC_TILE);
      const int qrow = static_cast<int>(base) + qb * TC_B;
      tma_load_2d(smem + TcSmem::Q, &tmQK, h * TC_HD, qrow, q_full);
      tma_load_2d(smem + TcSmem::Q + TC_HALF, &tmQK, h * TC_HD + 64, qrow, q_full);
      uint32_t it = 0;
      for (int kb = 0; kb <= qb && !*abort_flag; ++kb) {
        if (tc_state128(st64, nb64, qb, kb) == 0) continue;
        const int s = it & 1;
        if (!mbar_wait(&kv_empty[s], ((it >> 1) & 1) ^ 1)) {
          atomicMax(status, ST_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        const int krow = static_cast<int>(base) + kb * TC_B;
        uint8_t* sk = smem + TcSmem::K + s * TC_TILE;
        uint8_t* sv = smem + TcSmem::V + s * TC_TILE;
        mbar_expect_tx(&k_full[s], TC_TILE);
        tma_load_2d(sk, &tmQK, (Hq + kvh) * TC_HD, krow, &k_full[s]);
        tma_load_2d(sk + TC_HALF, &tmQK, (Hq + kvh) * TC_HD + 64, krow, &k_full[s]);
        mbar_expect_tx(&v_full[s], TC_TILE);
        tma_load_2d(sv, &tmVt, krow, kvh * TC_HD, &v_full[s]);
        tma_load_2d(sv + TC_HALF, &tmVt, krow + 64, kvh * TC_HD, &v_full[s]);
        ++it;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(TC_B, TC_B);
      const uint32_t sq = smem_u32(smem + TcSmem::Q), sp = smem_u32(smem + TcSmem::P);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) {
        atomicMax(status, ST_TIMEOUT_FULL);
        *abort_flag = 1;
      }
      auto issue_pv = [&](uint32_t i) -> bool {
        const int s = i & 1;
        const uint32_t ph = (i >> 1) & 1;
        if (!mbar_wait(&v_full[s], ph) || !mbar_wait(p_full, i & 1) || !mbar_wait(&pv_empty[s], ph ^ 1)) return false;
        tc_fence_after_sync();
        const uint32_t sv = smem_u32(smem + TcSmem::V + s * TC_TILE);
        const uint32_t d = tmem + 256 + s * TC_B;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) tc_mma_f16(d, tc_desc(sp, kk), tc_desc(sv, kk), idesc, kk != 0);
        tc_commit(&pv_full[s]);
        tc_commit(&kv_empty[s]);
        tc_commit(p_empty);
        return true;
      };
      uint32_t it = 0;
      for (int kb = 0; kb <= qb && ok && !*abort_flag; ++kb) {
        if (tc_state128(st64, nb64, qb, kb) == 0) continue;
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&k_full[s], ph) || !mbar_wait(&s_empty[s], ph ^ 1)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sk = smem_u32(smem + TcSmem::K + s * TC_TILE);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) tc_mma_f16(tmem + s * TC_B, tc_desc(sq, kk), tc_desc(sk, kk), idesc, kk != 0);
        tc_commit(&s_full[s]);
        if (it > 0 && !issue_pv(it - 1)) {
          ok = false;
          break;
        }
        ++it;
      }
      if (ok && !*abort_flag && it > 0 && !issue_pv(it - 1)) ok = false;
      if (!ok) {
        atomicMax(status, ST_TIMEOUT_TMEM_EMPTY);
        *abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / output warps
    // Two warps share each TMEM lane quarter: warp pair (q, half) handles columns [64*half, 64*half+64) of
    // the score rows 32q..32q+31 and the same half of the output columns.  The pair agrees on the row maximum
    // through shared memory and a two-arrival mbarrier per quarter.
    const int q = warp & 3;                 // TMEM lane quarter of this warp
    const int hf = (warp - 2) >> 2;         // which half of the columns
    const int r = q * 32 + lane;            // query row inside the tile
    int* gk = sGk + (q * 2 + hf) * 64;      // this warp's 64 key ids of a partially masked tile
    const long qi = base + qb * TC_B + r;
    const int gq = gid[qi], pq = pid[qi];
    const int qpos = qb * TC_B + r;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* prow = smem + TcSmem::P + hf * TC_HALF + r * 128;
    const int sw = r & 7;
    float O[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) O[i] = 0.f;
    float m = -INFINITY, l = 0.f, m_o = 0.f, ms_prev = 0.f;
    bool dead = false;
    uint32_t it = 0, xph = 0;

    auto fail = [&](int code) {
      if (lane == 0) {
        atomicMax(status, code);
        *abort_flag = 1;
      }
      dead = true;
    };
    // exchange one float with the partner thread (same row, other half); false on timeout
    auto swap_with_partner = [&](float mine, float& other) -> bool {
      float* slot = xch + (xph & 1) * 256;
      slot[hf * 128 + r] = mine;
      __syncwarp();
      if (lane == 0) mbar_arrive(&x_bar[q]);
      const int okw = mbar_wait(&x_bar[q], xph & 1) ? 1 : 0;
      if (!__all_sync(0xffffffffu, okw)) return false;
      other = slot[(hf ^ 1) * 128 + r];
      ++xph;
      return true;
    };
    auto add_pv = [&](uint32_t i, float ms_i) -> bool {
      const int s = i & 1;
      const int okw = mbar_wait(&pv_full[s], (i >> 1) & 1) ? 1 : 0;
      if (!__all_sync(0xffffffffu, okw)) return false;
      tc_fence_after_sync();
      const float f = ex2_approx(m_o - ms_i);
      m_o = ms_i;
#pragma unroll
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_off + 256 + s * TC_B + hf * 64 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) O[c + j] = fmaf(O[c + j], f, __uint_as_float(v[j]));
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pv_empty[s]);
      return true;
    };

    for (int kb = 0; kb <= qb; ++kb) {
      const int stt = tc_state128(st64, nb64, qb, kb);
      if (stt == 0) continue;
      if (__shfl_sync(0xffffffffu, *abort_flag, 0)) {
        dead = true;
        break;
      }
      const int s = it & 1;
      const bool partial = stt == 1;
      if (partial) {
        __syncwarp();
        gk[lane] = gid[base + kb * TC_B + hf * 64 + lane];
        gk[lane + 32] = gid[base + kb * TC_B + hf * 64 + lane + 32];
        __syncwarp();
      }
      const int okw = mbar_wait(&s_full[s], (it >> 1) & 1) ? 1 : 0;
      if (!__all_sync(0xffffffffu, okw)) {
        fail(ST_TIMEOUT_TMEM_FULL);
        break;
      }
      tc_fence_after_sync();
      // my half row of scores stays in registers from the max to the exponentials (single TMEM read)
      float x[64];
      {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(tmem + lane_off + s * TC_B + hf * 64, v0);
        tmem_ld_32x32(tmem + lane_off + s * TC_B + hf * 64 + 32, v1);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          x[j] = __uint_as_float(v0[j]);
          x[32 + j] = __uint_as_float(v1[j]);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
      if (partial) {
        const int k0 = kb * TC_B + hf * 64;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const int g = gk[j];
          if (!(k0 + j <= qpos && (g == gq || g == pq))) x[j] = -INFINITY;
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 64; ++j) mx4[j & 3] = fmaxf(mx4[j & 3], x[j]);
      const float mx_mine = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;   // scale > 0
      float mx_other;
      if (!swap_with_partner(mx_mine, mx_other)) {
        fail(ST_TIMEOUT_PEER);
        break;
      }
      const float mn = fmaxf(m, fmaxf(mx_mine, mx_other));
      const float ms = mn == -INFINITY ? 0.f : mn;
      l *= ex2_approx(m - ms);
      m = mn;
      // the previous tile's PV product has left shared memory P free once it was consumed
      const int okp = mbar_wait(p_empty, (it & 1) ^ 1) ? 1 : 0;
      if (!__all_sync(0xffffffffu, okp)) {
        fail(ST_TIMEOUT_EMPTY);
        break;
      }
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float pe[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          pe[e] = ex2_approx(fmaf(x[8 * i + e], scale_log2, -ms));
          rs4[e & 3] += pe[e];
        }
        uint4 w;
        w.x = pack_bf16x2(pe[0], pe[1]);
        w.y = pack_bf16x2(pe[2], pe[3]);
        w.z = pack_bf16x2(pe[4], pe[5]);
        w.w = pack_bf16x2(pe[6], pe[7]);
        *reinterpret_cast<uint4*>(prow + ((i ^ sw) << 4)) = w;
      }
      l += (rs4[0] + rs4[1]) + (rs4[2] + rs4[3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      // fold in the PV product of the previous tile while the tensor core works on this one
      if (it > 0 && !add_pv(it - 1, ms_prev)) {
        fail(ST_TIMEOUT_TMEM_FULL);
        break;
      }
      ms_prev = ms;
      ++it;
    }
    if (!dead && it > 0 && !add_pv(it - 1, ms_prev)) fail(ST_TIMEOUT_TMEM_FULL);
    float l_other = 0.f;
    if (!dead && !swap_with_partner(l, l_other)) fail(ST_TIMEOUT_PEER);
    if (!dead) {
      const float lt = l + l_other;
      const float inv = lt > 0.f ? 1.f / lt : 0.f;
      __nv_bfloat16* o = out + qi * ldo + h * TC_HD + hf * 64;
#pragma unroll
      for (int c = 0; c < 64; c += 8) {
        uint4 w;
        w.x = pack_bf16x2(O[c] * inv, O[c + 1] * inv);
        w.y = pack_bf16x2(O[c + 2] * inv, O[c + 3] * inv);
        w.z = pack_bf16x2(O[c + 4] * inv, O[c + 5] * inv);
        w.w = pack_bf16x2(O[c + 6] * inv, O[c + 7] * inv);
        *reinterpret_cast<uint4*>(o + c) = w;
      }
      if (hf == 0) lse2[static_cast<long>(h) * M + qi] = m + log2f(lt);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem, 512);
  }
}

// Vt[(kvh * 128 + d), token] = qkv[token, (Hq + Hkv + kvh) * 128 + d]
__global__ void attn_tc_transpose_v_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, int vcol0,
                                           __nv_bfloat16* __restrict__ vt, long M, int width) {
  __shared__ __nv_bfloat16 tile[32][33];
  const long t0 = static_cast<long>(blockIdx.x) * 32;
  const int c0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const long t = t0 + i;
    tile[i][threadIdx.x] = (t < M && c0 + static_cast<int>(threadIdx.x) < width)
                               ? qkv[t * ld + vcol0 + c0 + threadIdx.x]
                               : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i;
    const long t = t0 + threadIdx.x;
    if (c < width && t < M) vt[static_cast<size_t>(c) * M + t] = tile[threadIdx.x][i];
  }
}

}  // namespace artb

using namespace artb;

// qkv [rows*S, ld] post-RoPE, head dim 128, S % 128 == 0; vt: scratch bf16 [Hkv*128, rows*S]; state: the
// 64 x 64 tile-state table of artb_attn_tile_states; out [rows*S, Hq*128]; lse2 [Hq, rows*S].
ARTB_EXPORT int artb_attn_tc_fwd(const void* qkv, int ld, const int* gid, const int* pid, const uint8_t* state,
                                 void* vt, void* out, int ldo, float* lse2, int rows, int S, int Hq, int Hkv,
                                 int* status, cudaStream_t st) {
  if (S % TC_B || Hq % Hkv || (ld & 7) || (ldo & 7)) return ERR_BAD_SHAPE;
  const long M = static_cast<long>(rows) * S;
  if (M > 0x7fffffffL || (M & 7)) return ERR_BAD_SHAPE;
  {
    dim3 grid(static_cast<unsigned>((M + 31) / 32), (Hkv * TC_HD + 31) / 32), block(32, 8);
    attn_tc_transpose_v_kernel<<<grid, block, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(qkv), ld,
                                                       (Hq + Hkv) * TC_HD, reinterpret_cast<__nv_bfloat16*>(vt), M,
                                                       Hkv * TC_HD);
  }
  CUtensorMap tmQK, tmVt;
  int e;
  if ((e = make_tmap_bf16_2d(&tmQK, qkv, M, (Hq + 2 * Hkv) * TC_HD, ld, TC_B, 64))) return e;
  if ((e = make_tmap_bf16_2d(&tmVt, vt, static_cast<uint64_t>(Hkv) * TC_HD, M, M, TC_HD, 64))) return e;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t ce = cudaFuncSetAttribute(attn_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TcSmem::TOTAL);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    configured[dev & 63] = true;
  }
  const float scale_log2 = 1.4426950408889634f / sqrtf(static_cast<float>(TC_HD));
  dim3 grid(S / TC_B, Hq, rows);
  attn_tc_fwd_kernel<<<grid, TC_THREADS, TcSmem::TOTAL, st>>>(tmQK, tmVt, gid, pid, state,
                                                              reinterpret_cast<__nv_bfloat16*>(out), ldo, lse2, S, Hq,
                                                              Hkv, scale_log2, M, status);
  return static_cast<int>(cudaGetLastError());
}
