// Tree-masked flash attention backward on tcgen05 / TMEM (head dim 128), two kernels without atomics.
//
//   dkv kernel  one CTA per (128-key block, kv head); items = (query head of the group, 64-query block):
//       S^T  = K Q^T            UMMA 128 x 64 x 128   A = K tile (resident)   B = Q tile
//       dP^T = V dO^T           UMMA 128 x 64 x 128   A = V tile (resident)   B = dO tile
//       P^T  = exp2(S^T c - lse),  dS^T = c' P^T (dP^T - D)      thread = key row (TMEM lane), bf16 rows
//                                                                 written to shared memory, swizzled K-major
//       dV  += P^T dO           UMMA 128 x 128 x 64   A = P^T        B = dO^T tile (pre-transposed copy)
//       dK  += dS^T Q           UMMA 128 x 128 x 64   A = dS^T       B = Q^T tile  (pre-transposed copy)
//     dK and dV accumulate in TMEM over every item (all query heads of the group), so GQA needs no atomics.
//   dq kernel   one CTA per (128-query block, query head); items = 64-key blocks:
//       S = Q K^T,  dP = dO V^T  (128 x 64 x 128),  dS = c' P (dP - D)  thread = query row,
//       dQ += dS K               UMMA 128 x 128 x 64   A = dS   B = K^T tile (pre-transposed copy)
//
// Every operand is K-major with the 128-byte swizzle (the layout TMA writes and the only one this code base
// has validated); the three transposed copies (Q^T, dO^T, K^T: ~125 MB per layer at 8192 tokens) cost ~0.05 ms
// and remove the need for MN-major descriptors.  Both kernels recompute S (7 GEMM units instead of the
// minimal 5) in exchange for no fp32 dQ accumulator, no atomics and no conversion pass.
// TMEM: score buffers double-buffered (2 x 64 + 2 x 64 columns) + 128 or 256 accumulator columns.
// All waits are bounded; on expiry the CTA records a status code and unwinds.
//
// Reference semantics: autograd through SDPA with the dense bias of src/art/local/train.py:177-215.
#include <cuda_bf16.h>

#include <algorithm>

#include "host_utils.h"
#include "ptx_sm100.cuh"

namespace artb {

constexpr int TB_HD = 128;
constexpr int TB_THREADS = 576;   // TMA warp, MMA warp, 16 element-wise warps (four per TMEM lane quarter)

__device__ __forceinline__ float tb_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// [128 rows x 128 cols] tile as two 16 KB halves; [64 rows x 128 cols] tile as two 8 KB halves; k-step of 16 columns
__device__ __forceinline__ uint64_t tb_desc_r128(uint32_t base, int kk) {
  return umma_smem_desc_k128(base + (kk >> 2) * 16384) + 2 * (kk & 3);
}
__device__ __forceinline__ uint64_t tb_desc_r64(uint32_t base, int kk) {
  return umma_smem_desc_k128(base + (kk >> 2) * 8192) + 2 * (kk & 3);
}
// [128 rows x 64 cols] tile (one swizzle atom wide), k-step kk in 0..3
__device__ __forceinline__ uint64_t tb_desc_c64(uint32_t base, int kk) { return umma_smem_desc_k128(base) + 2 * kk; }

// ============================================================================================ dK / dV
struct DkvSmem {
  static constexpr int K = 0, V = 32768;
  static constexpr int STAGE = 65536;              // [2] x { Q 16K | dO 16K | Q^T 16K | dO^T 16K }
  static constexpr int PT = STAGE + 2 * 65536;     // P^T  [128 x 64] bf16
  static constexpr int DST = PT + 16384;           // dS^T [128 x 64] bf16
  static constexpr int LD = DST + 16384;           // float2 [16 warps][16]: (lse2, D) of the warp's 16 queries
  static constexpr int BAR = LD + 4 * 64 * 8;
  static constexpr int TOTAL = BAR + 256;          // 231 680 B; the dynamic window must start 1024-aligned
};

__global__ void __launch_bounds__(TB_THREADS, 1)
attn_tc_dkv_kernel(const __grid_constant__ CUtensorMap tmQKV128, const __grid_constant__ CUtensorMap tmQKV64,
                   const __grid_constant__ CUtensorMap tmDO64, const __grid_constant__ CUtensorMap tmQt,
                   const __grid_constant__ CUtensorMap tmDOt, const int* __restrict__ gid, const int* __restrict__ pid,
                   const uint8_t* __restrict__ state, const float* __restrict__ lse2, const float* __restrict__ Dv,
                   __nv_bfloat16* __restrict__ dqkv, int ld, int S, int Hq, int Hkv, float scale, float scale_log2, long M,
                   int GS, float* __restrict__ partial, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DkvSmem::BAR);
  uint64_t* kv_full = bars;
  uint64_t* stage_full = bars + 1;    // [2]
  uint64_t* stage_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;        // [2]
  uint64_t* s_empty = bars + 7;       // [2]
  uint64_t* pt_full = bars + 9;
  uint64_t* pt_empty = bars + 10;
  uint64_t* acc_full = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int nb64 = S / 64;
  // The query heads of a kv group can be split over GS CTAs (shorter critical path for the key blocks near the
  // start of a row, which see every later query); each then writes an fp32 partial that a combine kernel sums.
  const int kb = blockIdx.x, kvh = blockIdx.y / GS, gs = blockIdx.y % GS, row = blockIdx.z;
  const int Gall = Hq / Hkv, Gper = (Gall + GS - 1) / GS;
  const int g_lo = gs * Gper;
  const int G = min(Gall, g_lo + Gper) - g_lo;          // query heads handled here: g_lo .. g_lo + G - 1
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long base = static_cast<long>(row) * S;
  const uint8_t* st64 = state + static_cast<size_t>(row) * nb64 * nb64;
  const int qb_lo = 2 * kb, n_qb = nb64 - qb_lo;      // 64-query blocks at or below the diagonal
  const int n_items = G * n_qb;
  // item -> (group head g, 64-query block qb); state of the (qb, 128-key block) tile: 0 skip, 1 partial, 2 full
  auto item_state = [&](int item, int& g, int& qb) {
    g = item / n_qb;
    qb = qb_lo + item % n_qb;
    const uint8_t* r = st64 + static_cast<size_t>(qb) * nb64 + 2 * kb;
    const int a = r[0], b = r[1];
    return (a | b) == 0 ? 0 : ((a == 2 && b == 2) ? 2 : 1);
  };

  if ((smem_u32(smem) & 1023u) != 0) {   // the swizzled layouts below need a 1024-byte aligned window
    if (threadIdx.x == 0) atomicMax(status, ST_BAD_ARGS);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&stage_full[i], 1);
      mbar_init(&stage_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 16);
    }
    mbar_init(pt_full, 16);
    mbar_init(pt_empty, 1);
    mbar_init(acc_full, 1);
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
    if (lane == 0) {
      const int krow = static_cast<int>(base) + kb * 128;
      mbar_expect_tx(kv_full, 65536);
      tma_load_2d(smem + DkvSmem::K, &tmQKV128, (Hq + kvh) * TB_HD, krow, kv_full);
      tma_load_2d(smem + DkvSmem::K + 16384, &tmQKV128, (Hq + kvh) * TB_HD + 64, krow, kv_full);
      tma_load_2d(smem + DkvSmem::V, &tmQKV128, (Hq + Hkv + kvh) * TB_HD, krow, kv_full);
      tma_load_2d(smem + DkvSmem::V + 16384, &tmQKV128, (Hq + Hkv + kvh) * TB_HD + 64, krow, kv_full);
      uint32_t it = 0;
      for (int item = 0; item < n_items && !*abort_flag; ++item) {
        int g, qb;
        if (item_state(item, g, qb) == 0) continue;
        const int s = it & 1;
        if (!mbar_wait(&stage_empty[s], ((it >> 1) & 1) ^ 1)) {
          atomicMax(status, ST_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        const int hq = kvh * Gall + g_lo + g;
        const int qrow = static_cast<int>(base) + qb * 64;
        uint8_t* st = smem + DkvSmem::STAGE + s * 65536;
        mbar_expect_tx(&stage_full[s], 65536);
        tma_load_2d(st, &tmQKV64, hq * TB_HD, qrow, &stage_full[s]);
        tma_load_2d(st + 8192, &tmQKV64, hq * TB_HD + 64, qrow, &stage_full[s]);
        tma_load_2d(st + 16384, &tmDO64, hq * TB_HD, qrow, &stage_full[s]);
        tma_load_2d(st + 24576, &tmDO64, hq * TB_HD + 64, qrow, &stage_full[s]);
        tma_load_2d(st + 32768, &tmQt, qrow, hq * TB_HD, &stage_full[s]);
        tma_load_2d(st + 49152, &tmDOt, qrow, hq * TB_HD, &stage_full[s]);
        ++it;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t id_s = umma_idesc_bf16(128, 64), id_acc = umma_idesc_bf16(128, 128);
      const uint32_t sK = smem_u32(smem + DkvSmem::K), sV = smem_u32(smem + DkvSmem::V);
      const uint32_t sPT = smem_u32(smem + DkvSmem::PT), sDST = smem_u32(smem + DkvSmem::DST);
      bool ok = mbar_wait(kv_full, 0);
      auto issue_acc = [&](uint32_t i) -> bool {
        const int s = i & 1;
        if (!mbar_wait(pt_full, i & 1)) return false;
        tc_fence_after_sync();
        const uint32_t st = smem_u32(smem + DkvSmem::STAGE + s * 65536);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tc_mma_f16(tmem + 256, tb_desc_c64(sPT, kk), tb_desc_c64(st + 49152, kk), id_acc, (i | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tc_mma_f16(tmem + 384, tb_desc_c64(sDST, kk), tb_desc_c64(st + 32768, kk), id_acc, (i | kk) != 0);
        tc_commit(&stage_empty[s]);
        tc_commit(pt_empty);
        return true;
      };
      uint32_t it = 0;
      for (int item = 0; item < n_items && ok && !*abort_flag; ++item) {
        int g, qb;
        if (item_state(item, g, qb) == 0) continue;
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&stage_full[s], ph) || !mbar_wait(&s_empty[s], ph ^ 1)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t st = smem_u32(smem + DkvSmem::STAGE + s * 65536);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tc_mma_f16(tmem + s * 64, tb_desc_r128(sK, kk), tb_desc_r64(st, kk), id_s, kk != 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tc_mma_f16(tmem + 128 + s * 64, tb_desc_r128(sV, kk), tb_desc_r64(st + 16384, kk), id_s, kk != 0);
        tc_commit(&s_full[s]);
        if (it > 0 && !issue_acc(it - 1)) {
          ok = false;
          break;
        }
        ++it;
      }
      if (ok && !*abort_flag && it > 0 && !issue_acc(it - 1)) ok = false;
      if (!ok) {
        atomicMax(status, ST_TIMEOUT_FULL);
        *abort_flag = 1;
      }
      tc_commit(acc_full);
    }
  } else {
    // thread = (key row r, column quarter hf): 16 of the item's 64 query columns; four warps share a TMEM lane
    // quarter, which gives every scheduler four element-wise warps to overlap TMEM / MUFU / shared-memory latency
    const int q = warp & 3, hf = (warp - 2) >> 2;
    const int r = q * 32 + lane;                 // key row inside the block
    const long ki = base + kb * 128 + r;
    const int gk_mine = gid[ki];
    const int kpos = kb * 128 + r;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    float2* ldw = reinterpret_cast<float2*>(smem + DkvSmem::LD) + (q * 4 + hf) * 16;   // (lse2, D) of my 16 queries
    uint8_t* pt_row = smem + DkvSmem::PT + r * 128;
    uint8_t* dst_row = smem + DkvSmem::DST + r * 128;
    const int sw = r & 7;
    const int l16 = lane & 15;
    bool dead = false;
    uint32_t it = 0;
    // items are visited in (g, qb) order; the per-query constants of the NEXT valid item are fetched from global
    // memory one item ahead so that their latency is off the critical path
    auto next_valid = [&](int& g, int& qb) {      // advance (g, qb) to the next non-empty item; false at the end
      for (;;) {
        if (++qb >= nb64) {
          qb = qb_lo;
          if (++g >= G) return false;
        }
        const uint8_t* sr = st64 + static_cast<size_t>(qb) * nb64 + 2 * kb;
        if ((sr[0] | sr[1]) != 0) return true;
      }
    };
    auto fetch = [&](int g, int qb, float2& ld, int& gq, int& pq) {
      const long qidx = base + qb * 64 + hf * 16 + l16;
      const long hidx = static_cast<long>(kvh * Gall + g_lo + g) * M + qidx;
      ld = make_float2(lse2[hidx], Dv[hidx]);
      gq = gid[qidx];
      pq = pid[qidx];
    };
    int g = 0, qb = qb_lo - 1;
    bool have = G > 0 && next_valid(g, qb);
    float2 ld_cur = make_float2(0.f, 0.f);
    int gq_cur = 0, pq_cur = 0;
    if (have) fetch(g, qb, ld_cur, gq_cur, pq_cur);
    while (have) {
      if (__shfl_sync(0xffffffffu, *abort_flag, 0)) {
        dead = true;
        break;
      }
      const uint8_t* sr = st64 + static_cast<size_t>(qb) * nb64 + 2 * kb;
      const bool partial = !(sr[0] == 2 && sr[1] == 2);
      const int qpos0 = qb * 64 + hf * 16;
      const int s = it & 1;
      __syncwarp();
      if (lane < 16) ldw[lane] = ld_cur;
      const int gq_h = gq_cur, pq_h = pq_cur;
      int g2 = g, qb2 = qb;
      const bool have2 = next_valid(g2, qb2);
      if (have2) fetch(g2, qb2, ld_cur, gq_cur, pq_cur);   // in flight while this item is processed
      __syncwarp();
      const int okw = mbar_wait(&s_full[s], (it >> 1) & 1) ? 1 : 0;
      if (!__all_sync(0xffffffffu, okw)) {
        if (lane == 0) {
          atomicMax(status, ST_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        dead = true;
        break;
      }
      tc_fence_after_sync();
      uint32_t xs[16], xd[16];   // S^T and dP^T of my key row, my 16 query columns
      tmem_ld_32x16(tmem + lane_off + s * 64 + hf * 16, xs);
      tmem_ld_32x16(tmem + lane_off + 128 + s * 64 + hf * 16, xd);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
      const float4* ld4 = reinterpret_cast<const float4*>(ldw);
      uint4 w[2], v[2];
#pragma unroll
      for (int ii = 0; ii < 2; ++ii) {
        float pe[8], de[8];
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const int jj = 8 * ii + e;
          const float4 l4 = ld4[jj >> 1];      // (lse, D) of queries jj and jj + 1
          float p0 = tb_ex2(fmaf(__uint_as_float(xs[jj]), scale_log2, -l4.x));
          float p1 = tb_ex2(fmaf(__uint_as_float(xs[jj + 1]), scale_log2, -l4.z));
          if (partial) {
            const int g0 = __shfl_sync(0xffffffffu, gq_h, jj), q0i = __shfl_sync(0xffffffffu, pq_h, jj);
            const int g1 = __shfl_sync(0xffffffffu, gq_h, jj + 1), q1i = __shfl_sync(0xffffffffu, pq_h, jj + 1);
            if (!(kpos <= qpos0 + jj && (gk_mine == g0 || gk_mine == q0i))) p0 = 0.f;
            if (!(kpos <= qpos0 + jj + 1 && (gk_mine == g1 || gk_mine == q1i))) p1 = 0.f;
          }
          pe[e] = p0;
          pe[e + 1] = p1;
          de[e] = p0 * (__uint_as_float(xd[jj]) - l4.y);          // the softmax scale is applied to dK at the end
          de[e + 1] = p1 * (__uint_as_float(xd[jj + 1]) - l4.w);
        }
        w[ii].x = pack_bf16x2(pe[0], pe[1]);
        w[ii].y = pack_bf16x2(pe[2], pe[3]);
        w[ii].z = pack_bf16x2(pe[4], pe[5]);
        w[ii].w = pack_bf16x2(pe[6], pe[7]);
        v[ii].x = pack_bf16x2(de[0], de[1]);
        v[ii].y = pack_bf16x2(de[2], de[3]);
        v[ii].z = pack_bf16x2(de[4], de[5]);
        v[ii].w = pack_bf16x2(de[6], de[7]);
      }
      // only now wait for the previous item's accumulate MMAs to release the P^T / dS^T tiles
      const int okp = mbar_wait(pt_empty, (it & 1) ^ 1) ? 1 : 0;
      if (!__all_sync(0xffffffffu, okp)) {
        if (lane == 0) {
          atomicMax(status, ST_TIMEOUT_EMPTY);
          *abort_flag = 1;
        }
        dead = true;
        break;
      }
#pragma unroll
      for (int ii = 0; ii < 2; ++ii) {
        const int piece = 2 * hf + ii;
        *reinterpret_cast<uint4*>(pt_row + ((piece ^ sw) << 4)) = w[ii];
        *reinterpret_cast<uint4*>(dst_row + ((piece ^ sw) << 4)) = v[ii];
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pt_full);
      ++it;
      g = g2;
      qb = qb2;
      have = have2;
    }
    // accumulators -> dK, dV rows of this key block (bf16 into the fused gradient buffer); my 32 columns of each
    if (!dead) {
      const int okw = mbar_wait(acc_full, 0) ? 1 : 0;
      if (!__all_sync(0xffffffffu, okw)) {
        if (lane == 0) {
          atomicMax(status, ST_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        dead = true;
      }
    }
    if (!dead) {
      tc_fence_after_sync();
      __nv_bfloat16* dk = dqkv + ki * ld + (Hq + kvh) * TB_HD + hf * 32;
      __nv_bfloat16* dv = dqkv + ki * ld + (Hq + Hkv + kvh) * TB_HD + hf * 32;
      // partial layout: fp32 [GS][M][2 * Hkv * 128], columns = dk of all kv heads, then dv of all kv heads
      float* pk = partial ? partial + (static_cast<size_t>(gs) * M + ki) * (2 * Hkv * TB_HD) + kvh * TB_HD + hf * 32 : nullptr;
      float* pv = partial ? pk + Hkv * TB_HD : nullptr;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* o = which == 0 ? dv : dk;
        float* po = which == 0 ? pv : pk;
        const float f = which == 0 ? 1.f : scale;
        const uint32_t col0 = 256 + which * 128 + hf * 32;
#pragma unroll 1
        for (int c = 0; c < 32; c += 32) {
          uint32_t v[32];
          if (it > 0) {
            tmem_ld_32x32(tmem + lane_off + col0 + c, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
          if (po) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) *reinterpret_cast<uint4*>(po + c + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            continue;
          }
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(v[j]) * f, __uint_as_float(v[j + 1]) * f);
            w.y = pack_bf16x2(__uint_as_float(v[j + 2]) * f, __uint_as_float(v[j + 3]) * f);
            w.z = pack_bf16x2(__uint_as_float(v[j + 4]) * f, __uint_as_float(v[j + 5]) * f);
            w.w = pack_bf16x2(__uint_as_float(v[j + 6]) * f, __uint_as_float(v[j + 7]) * f);
            *reinterpret_cast<uint4*>(o + c + j) = w;
          }
        }
      }
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

// ================================================================================================= dQ
struct DqSmem {
  static constexpr int Q = 0, DO = 32768;
  static constexpr int STAGE = 65536;              // [2] x { K 16K | V 16K | K^T 16K }
  static constexpr int DS = STAGE + 2 * 49152;     // [2] x dS [128 x 64] bf16
  static constexpr int GK = DS + 2 * 16384;        // int [16 warps][16]
  static constexpr int BAR = GK + 4 * 64 * 4;
  static constexpr int TOTAL = BAR + 256;
};

__global__ void __launch_bounds__(TB_THREADS, 1)
attn_tc_dq_kernel(const __grid_constant__ CUtensorMap tmQKV128, const __grid_constant__ CUtensorMap tmQKV64,
                  const __grid_constant__ CUtensorMap tmDO128, const __grid_constant__ CUtensorMap tmKt,
                  const int* __restrict__ gid, const int* __restrict__ pid, const uint8_t* __restrict__ state,
                  const float* __restrict__ lse2, const float* __restrict__ Dv, __nv_bfloat16* __restrict__ dqkv, int ld,
                  int S, int Hq, int Hkv, float scale, float scale_log2, long M, int* status) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DqSmem::BAR);
  uint64_t* qdo_full = bars;
  uint64_t* stage_full = bars + 1;    // [2]
  uint64_t* stage_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;        // [2]
  uint64_t* s_empty = bars + 7;       // [2]
  uint64_t* ds_full = bars + 9;       // [2]
  uint64_t* ds_empty = bars + 11;     // [2]
  uint64_t* acc_full = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int nb = S / 128, nb64 = S / 64;
  const int qb = nb - 1 - blockIdx.x, h = blockIdx.y, row = blockIdx.z;
  const int kvh = h / (Hq / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long base = static_cast<long>(row) * S;
  const uint8_t* st64 = state + static_cast<size_t>(row) * nb64 * nb64;
  const int n_items = 2 * qb + 2;          // 64-key blocks at or below the diagonal
  auto item_state = [&](int kb64) {
    const int a = st64[static_cast<size_t>(2 * qb) * nb64 + kb64], b = st64[static_cast<size_t>(2 * qb + 1) * nb64 + kb64];
    return (a | b) == 0 ? 0 : ((a == 2 && b == 2) ? 2 : 1);
  };

  if ((smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0) atomicMax(status, ST_BAD_ARGS);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&stage_full[i], 1);
      mbar_init(&stage_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 16);
      mbar_init(&ds_full[i], 16);
      mbar_init(&ds_empty[i], 1);
    }
    mbar_init(acc_full, 1);
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
    if (lane == 0) {
      const int qrow = static_cast<int>(base) + qb * 128;
      mbar_expect_tx(qdo_full, 65536);
      tma_load_2d(smem + DqSmem::Q, &tmQKV128, h * TB_HD, qrow, qdo_full);
      tma_load_2d(smem + DqSmem::Q + 16384, &tmQKV128, h * TB_HD + 64, qrow, qdo_full);
      tma_load_2d(smem + DqSmem::DO, &tmDO128, h * TB_HD, qrow, qdo_full);
      tma_load_2d(smem + DqSmem::DO + 16384, &tmDO128, h * TB_HD + 64, qrow, qdo_full);
      uint32_t it = 0;
      for (int kb = 0; kb < n_items && !*abort_flag; ++kb) {
        if (item_state(kb) == 0) continue;
        const int s = it & 1;
        if (!mbar_wait(&stage_empty[s], ((it >> 1) & 1) ^ 1)) {
          atomicMax(status, ST_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        const int krow = static_cast<int>(base) + kb * 64;
        uint8_t* st = smem + DqSmem::STAGE + s * 49152;
        mbar_expect_tx(&stage_full[s], 49152);
        tma_load_2d(st, &tmQKV64, (Hq + kvh) * TB_HD, krow, &stage_full[s]);
        tma_load_2d(st + 8192, &tmQKV64, (Hq + kvh) * TB_HD + 64, krow, &stage_full[s]);
        tma_load_2d(st + 16384, &tmQKV64, (Hq + Hkv + kvh) * TB_HD, krow, &stage_full[s]);
        tma_load_2d(st + 24576, &tmQKV64, (Hq + Hkv + kvh) * TB_HD + 64, krow, &stage_full[s]);
        tma_load_2d(st + 32768, &tmKt, krow, kvh * TB_HD, &stage_full[s]);
        ++it;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t id_s = umma_idesc_bf16(128, 64), id_acc = umma_idesc_bf16(128, 128);
      const uint32_t sQ = smem_u32(smem + DqSmem::Q), sDO = smem_u32(smem + DqSmem::DO);
      bool ok = mbar_wait(qdo_full, 0);
      auto issue_acc = [&](uint32_t i) -> bool {
        const int s = i & 1;
        if (!mbar_wait(&ds_full[s], (i >> 1) & 1)) return false;
        tc_fence_after_sync();
        const uint32_t st = smem_u32(smem + DqSmem::STAGE + s * 49152);
        const uint32_t sds = smem_u32(smem + DqSmem::DS + s * 16384);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          tc_mma_f16(tmem + 256, tb_desc_c64(sds, kk), tb_desc_c64(st + 32768, kk), id_acc, (i | kk) != 0);
        tc_commit(&stage_empty[s]);
        tc_commit(&ds_empty[s]);
        return true;
      };
      uint32_t it = 0;
      for (int kb = 0; kb < n_items && ok && !*abort_flag; ++kb) {
        if (item_state(kb) == 0) continue;
        const int s = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&stage_full[s], ph) || !mbar_wait(&s_empty[s], ph ^ 1)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t st = smem_u32(smem + DqSmem::STAGE + s * 49152);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tc_mma_f16(tmem + s * 64, tb_desc_r128(sQ, kk), tb_desc_r64(st, kk), id_s, kk != 0);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          tc_mma_f16(tmem + 128 + s * 64, tb_desc_r128(sDO, kk), tb_desc_r64(st + 16384, kk), id_s, kk != 0);
        tc_commit(&s_full[s]);
        if (it > 0 && !issue_acc(it - 1)) {
          ok = false;
          break;
        }
        ++it;
      }
      if (ok && !*abort_flag && it > 0 && !issue_acc(it - 1)) ok = false;
      if (!ok) {
        atomicMax(status, ST_TIMEOUT_FULL);
        *abort_flag = 1;
      }
      tc_commit(acc_full);
    }
  } else {
    // thread = (query row r, column quarter hf): 16 of the item's 64 key columns
    const int q = warp & 3, hf = (warp - 2) >> 2;
    const int r = q * 32 + lane;                 // query row inside the block
    const long qi = base + qb * 128 + r;
    const int gq = gid[qi], pq = pid[qi];
    const int qpos = qb * 128 + r;
    const float lse_r = lse2[static_cast<long>(h) * M + qi], D_r = Dv[static_cast<long>(h) * M + qi];
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    int* gk = reinterpret_cast<int*>(smem + DqSmem::GK) + (q * 4 + hf) * 16;
    const int sw = r & 7;
    bool dead = false;
    uint32_t it = 0;
    for (int kb = 0; kb < n_items; ++kb) {
      const int stt = item_state(kb);
      if (stt == 0) continue;
      if (__shfl_sync(0xffffffffu, *abort_flag, 0)) {
        dead = true;
        break;
      }
      const int s = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const bool partial = stt == 1;
      if (partial) {
        __syncwarp();
        if (lane < 16) gk[lane] = gid[base + kb * 64 + hf * 16 + lane];
        __syncwarp();
      }
      const int okw = mbar_wait(&s_full[s], ph) ? 1 : 0;
      if (!__all_sync(0xffffffffu, okw)) {
        if (lane == 0) {
          atomicMax(status, ST_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        dead = true;
        break;
      }
      tc_fence_after_sync();
      uint32_t xs[16], xd[16];   // S and dP of my query row, my 16 key columns
      tmem_ld_32x16(tmem + lane_off + s * 64 + hf * 16, xs);
      tmem_ld_32x16(tmem + lane_off + 128 + s * 64 + hf * 16, xd);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
      const int okp = mbar_wait(&ds_empty[s], ph ^ 1) ? 1 : 0;
      if (!__all_sync(0xffffffffu, okp)) {
        if (lane == 0) {
          atomicMax(status, ST_TIMEOUT_EMPTY);
          *abort_flag = 1;
        }
        dead = true;
        break;
      }
      uint8_t* ds_row = smem + DqSmem::DS + s * 16384 + r * 128;
      const int k0 = kb * 64 + hf * 16;
#pragma unroll
      for (int ii = 0; ii < 2; ++ii) {
        float de[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int jj = 8 * ii + e;
          float p = tb_ex2(fmaf(__uint_as_float(xs[jj]), scale_log2, -lse_r));
          if (partial) {
            const int g = gk[jj];
            if (!(k0 + jj <= qpos && (g == gq || g == pq))) p = 0.f;
          }
          de[e] = p * (__uint_as_float(xd[jj]) - D_r);            // the softmax scale is applied to dQ at the end
        }
        uint4 v;
        v.x = pack_bf16x2(de[0], de[1]);
        v.y = pack_bf16x2(de[2], de[3]);
        v.z = pack_bf16x2(de[4], de[5]);
        v.w = pack_bf16x2(de[6], de[7]);
        *reinterpret_cast<uint4*>(ds_row + (((2 * hf + ii) ^ sw) << 4)) = v;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[s]);
      ++it;
    }
    if (!dead) {
      const int okw = mbar_wait(acc_full, 0) ? 1 : 0;
      if (!__all_sync(0xffffffffu, okw)) {
        if (lane == 0) {
          atomicMax(status, ST_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        dead = true;
      }
    }
    if (!dead) {
      tc_fence_after_sync();
      __nv_bfloat16* o = dqkv + qi * ld + h * TB_HD + hf * 32;
#pragma unroll 1
      for (int c = 0; c < 32; c += 32) {
        uint32_t v[32];
        if (it > 0) {
          tmem_ld_32x32(tmem + lane_off + 256 + hf * 32 + c, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 w;
          w.x = pack_bf16x2(__uint_as_float(v[j]) * scale, __uint_as_float(v[j + 1]) * scale);
          w.y = pack_bf16x2(__uint_as_float(v[j + 2]) * scale, __uint_as_float(v[j + 3]) * scale);
          w.z = pack_bf16x2(__uint_as_float(v[j + 4]) * scale, __uint_as_float(v[j + 5]) * scale);
          w.w = pack_bf16x2(__uint_as_float(v[j + 6]) * scale, __uint_as_float(v[j + 7]) * scale);
          *reinterpret_cast<uint4*>(o + c + j) = w;
        }
      }
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

// dk|dv rows = sum over the GS partials (dk scaled), written as bf16 into the k|v columns of dqkv
__global__ void attn_tc_combine_dkv_kernel(const float* __restrict__ partial, int GS, __nv_bfloat16* __restrict__ dqkv, int ld,
                                           int kcol0, long M, int kvw /* Hkv * 128 */, float scale) {
  const int vec = (2 * kvw) >> 2;
  const long total = M * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long m = i / vec;
    const int c = static_cast<int>(i % vec) * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int g = 0; g < GS; ++g) {
      const float4 v = *reinterpret_cast<const float4*>(partial + (static_cast<size_t>(g) * M + m) * (2 * kvw) + c);
      a.x += v.x;
      a.y += v.y;
      a.z += v.z;
      a.w += v.w;
    }
    const float f = c < kvw ? scale : 1.f;
    uint2 o;
    o.x = pack_bf16x2(a.x * f, a.y * f);
    o.y = pack_bf16x2(a.z * f, a.w * f);
    *reinterpret_cast<uint2*>(dqkv + m * ld + kcol0 + c) = o;
  }
}

// dst[c, token] = src[token, c0 + c] for c < width: 64 x 64 tiles, 16-byte loads and stores (M % 8 == 0, width % 64 == 0)
__global__ void __launch_bounds__(256)
attn_tc_transpose_kernel(const __nv_bfloat16* __restrict__ src, int ld, int c0, __nv_bfloat16* __restrict__ dst, long M,
                         int width) {
  __shared__ __nv_bfloat16 tile[64][64 + 8];
  const long t0 = static_cast<long>(blockIdx.x) * 64;
  const int cb = blockIdx.y * 64;
  const int tid = threadIdx.x;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int v = tid + i * 256;          // 512 vectors: 64 tokens x 8
    const int r = v >> 3, cv = v & 7;
    const long t = t0 + r;
    uint4 x = make_uint4(0, 0, 0, 0);
    if (t < M) x = *reinterpret_cast<const uint4*>(src + t * ld + c0 + cb + cv * 8);
    *reinterpret_cast<uint4*>(&tile[r][cv * 8]) = x;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int v = tid + i * 256;          // 512 vectors: 64 columns x 8 token groups
    const int c = v >> 3, tv = v & 7;
    __nv_bfloat16 e[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) e[j] = tile[tv * 8 + j][c];
    const long t = t0 + tv * 8;
    if (t < M) *reinterpret_cast<uint4*>(dst + static_cast<size_t>(cb + c) * M + t) = *reinterpret_cast<const uint4*>(e);
  }
}

// D[h, m] = sum_d dO[m, h*128 + d] * O[m, h*128 + d]   (one warp per (token, head))
__global__ void attn_tc_rowdot_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O, int ld,
                                      float* __restrict__ D, long M, int Hq) {
  const long wid = blockIdx.x * static_cast<long>(blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (wid >= M * Hq) return;
  const long m = wid / Hq;
  const int h = static_cast<int>(wid % Hq);
  const uint2 a = *reinterpret_cast<const uint2*>(dO + m * ld + h * TB_HD + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(O + m * ld + h * TB_HD + lane * 4);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
  const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) D[static_cast<long>(h) * M + m] = s;
}

}  // namespace artb

using namespace artb;

// qkv / dqkv [rows*S, ld] (q | k | v columns); out, dout [rows*S, ldo]; lse2, Dbuf fp32 [Hq, rows*S];
// scratch bf16: qt, dot [Hq*128, rows*S], kt [Hkv*128, rows*S]; partial: optional fp32 [2, rows*S, 2*Hkv*128]
// (enables the two-way split of a kv group's query heads).  Head dim 128, S % 128 == 0.
ARTB_EXPORT int artb_attn_tc_bwd(const void* qkv, int ld, const void* out, const void* dout, int ldo, const int* gid,
                                 const int* pid, const uint8_t* state, const float* lse2, float* Dbuf, void* qt, void* dot,
                                 void* kt, void* dqkv, float* partial, int rows, int S, int Hq, int Hkv, int* status,
                                 cudaStream_t st) {
  if (S % 128 || Hq % Hkv || (ld & 7) || (ldo & 7)) return ERR_BAD_SHAPE;
  const long M = static_cast<long>(rows) * S;
  if (M > 0x7fffffffL) return ERR_BAD_SHAPE;
  typedef __nv_bfloat16 bf;
  {
    const long warps = M * Hq;
    attn_tc_rowdot_kernel<<<static_cast<unsigned>((warps + 3) / 4), 128, 0, st>>>(
        reinterpret_cast<const bf*>(dout), reinterpret_cast<const bf*>(out), ldo, Dbuf, M, Hq);
    const unsigned block = 256;
    dim3 gq(static_cast<unsigned>((M + 63) / 64), Hq * TB_HD / 64), gk(static_cast<unsigned>((M + 63) / 64), Hkv * TB_HD / 64);
    attn_tc_transpose_kernel<<<gq, block, 0, st>>>(reinterpret_cast<const bf*>(qkv), ld, 0, reinterpret_cast<bf*>(qt), M,
                                                   Hq * TB_HD);
    attn_tc_transpose_kernel<<<gq, block, 0, st>>>(reinterpret_cast<const bf*>(dout), ldo, 0, reinterpret_cast<bf*>(dot), M,
                                                   Hq * TB_HD);
    attn_tc_transpose_kernel<<<gk, block, 0, st>>>(reinterpret_cast<const bf*>(qkv), ld, Hq * TB_HD,
                                                   reinterpret_cast<bf*>(kt), M, Hkv * TB_HD);
  }
  CUtensorMap tmQKV128, tmQKV64, tmDO128, tmDO64, tmQt, tmDOt, tmKt;
  int e;
  const uint64_t W = static_cast<uint64_t>(Hq + 2 * Hkv) * TB_HD;
  if ((e = make_tmap_bf16_2d(&tmQKV128, qkv, M, W, ld, 128, 64))) return e;
  if ((e = make_tmap_bf16_2d(&tmQKV64, qkv, M, W, ld, 64, 64))) return e;
  if ((e = make_tmap_bf16_2d(&tmDO128, dout, M, static_cast<uint64_t>(Hq) * TB_HD, ldo, 128, 64))) return e;
  if ((e = make_tmap_bf16_2d(&tmDO64, dout, M, static_cast<uint64_t>(Hq) * TB_HD, ldo, 64, 64))) return e;
  if ((e = make_tmap_bf16_2d(&tmQt, qt, static_cast<uint64_t>(Hq) * TB_HD, M, M, 128, 64))) return e;
  if ((e = make_tmap_bf16_2d(&tmDOt, dot, static_cast<uint64_t>(Hq) * TB_HD, M, M, 128, 64))) return e;
  if ((e = make_tmap_bf16_2d(&tmKt, kt, static_cast<uint64_t>(Hkv) * TB_HD, M, M, 128, 64))) return e;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t ce = cudaFuncSetAttribute(attn_tc_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvSmem::TOTAL);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    ce = cudaFuncSetAttribute(attn_tc_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem::TOTAL);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    configured[dev & 63] = true;
  }
  const float scale = 1.f / sqrtf(static_cast<float>(TB_HD));
  const float scale_log2 = 1.4426950408889634f * scale;
  // split the query heads of a group over two CTAs when a group has at least four heads and the caller gave scratch
  const int GS = (partial != nullptr && Hq / Hkv >= 4) ? 2 : 1;
  dim3 g1(S / 128, Hkv * GS, rows), g2(S / 128, Hq, rows);
  attn_tc_dkv_kernel<<<g1, TB_THREADS, DkvSmem::TOTAL, st>>>(tmQKV128, tmQKV64, tmDO64, tmQt, tmDOt, gid, pid, state, lse2,
                                                            Dbuf, reinterpret_cast<bf*>(dqkv), ld, S, Hq, Hkv, scale,
                                                            scale_log2, M, GS, GS > 1 ? partial : nullptr, status);
  if (GS > 1) {
    const long total = M * ((2 * Hkv * TB_HD) >> 2);
    attn_tc_combine_dkv_kernel<<<static_cast<unsigned>(std::min<long>((total + 255) / 256, 148 * 16)), 256, 0, st>>>(
        partial, GS, reinterpret_cast<bf*>(dqkv), ld, Hq * TB_HD, M, Hkv * TB_HD, scale);
  }
  attn_tc_dq_kernel<<<g2, TB_THREADS, DqSmem::TOTAL, st>>>(tmQKV128, tmQKV64, tmDO128, tmKt, gid, pid, state, lse2, Dbuf,
                                                          reinterpret_cast<bf*>(dqkv), ld, S, Hq, Hkv, scale, scale_log2,
                                                          M, status);
  return static_cast<int>(cudaGetLastError());
}
