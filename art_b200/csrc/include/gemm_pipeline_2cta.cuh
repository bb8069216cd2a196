// 2-CTA variant of the tcgen05 GEMM pipeline: a cluster of two CTAs computes one 256 x 256
// output tile with `tcgen05.mma.cta_group::2` (UMMA M = 256, N = 256, K = 16).
//
// Why: with one CTA per 128 x 256 tile every UMMA reads 4 KB of A and 8 KB of B from shared
// memory while TMA writes the same amount, which saturates the 128 B/clk shared-memory port.
// In a pair each CTA stages only its own 128 rows of A and its own 128-row half of B (the
// tensor core reads the other half from the partner's shared memory), so per-SM staging traffic
// drops by a third and the B panel is fetched from L2 once per pair.
//
// Protocol (rank 0 of the pair is the leader):
//   full[s]    leader only, count 1 (+ tx bytes of BOTH CTAs' loads; TMA uses .cta_group::2 so the
//              partner's loads credit the leader's barrier; no multicast qualifier anywhere)
//   empty[s]   in both CTAs, count 1, signalled by the leader's tcgen05.commit multicast to both
//   tfull[b]   in both CTAs, count 1, same multicast commit once a tile's MMAs are issued
//   tempty[b]  leader only, count 8 (16 with a column-split epilogue): the epilogue warps of each CTA arrive (the
//              partner's remotely)
// All waits are bounded; a timeout sets the CTA's abort flag and the status word, and the CTA
// falls through to the teardown (cluster barrier, TMEM dealloc).
#pragma once
#include "gemm_pipeline.cuh"

namespace artb {

// BN2 = cluster tile N (256, or 224 when that wastes less of the last wave); each CTA stages
// BN2 / 2 rows of B.  Stage sizes stay multiples of 1024 B (the 128-byte-swizzle atom).
template <int STAGES, int BN2>
struct Gemm2SmemLayout {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = (GEMM_BM + BN2 / 2) * GEMM_BK * 2;
  static_assert(STAGE_BYTES % 1024 == 0 && BN2 % 32 == 0 && BN2 <= 256, "2-CTA tile");
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int TOTAL = BAR_OFFSET + BAR_BYTES + 1024;
};

// Schedule of the plain and split-K CTA-pair GEMMs.  `m_blk` of the tiles it returns counts 256-row PAIR tiles (the
// kernel turns it into each CTA's 128-row index).  splits > 1: the K range of every output tile is cut into `splits`
// slices of kb_per blocks; a work item is (tile, slice) and its partial goes through an accumulating epilogue (no
// extra-K operands in that mode).
struct SchedPair {
  int m_tiles2, n_tiles, group_m, splits, kb_per, kb_main;
  __device__ int tiles_for_cta(int cluster, int nclusters) const {
    const int total = m_tiles2 * n_tiles * splits;
    return cluster < total ? (total - cluster + nclusters - 1) / nclusters : 0;
  }
  __device__ TileInfo get(int cluster, int nclusters, int i) const {
    const int tile = cluster + i * nclusters;
    const int mn_tiles = m_tiles2 * n_tiles;
    const int mn = tile % mn_tiles, sp = tile / mn_tiles;
    int m2, nb;
    raster_tile(mn, m_tiles2, n_tiles, group_m, m2, nb);
    TileInfo ti = make_tile(m2, nb);
    if (splits > 1) {
      ti.group = sp;
      ti.kb_lo = sp * kb_per;
      ti.kb_n = max(0, min(kb_per, kb_main - ti.kb_lo));
      ti.extra = 0;
    }
    return ti;
  }
};

// Sched: tiles in units of 256 x BN2 (see SchedPair); Epi / Comm: the same policies as the one-CTA pipeline, called
// per CTA with that CTA's 128-row tile index, so the fused tensor-parallel policies work unchanged (each CTA's producer
// waits for the arrival of its own 128 rows; each CTA's epilogue scatters / reduces its own 128 x BN2 half).
template <int STAGES, int BN2, class Sched, class Epi, class Comm = NoComm>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gemm_pipe_threads<Epi>() + Comm::THREADS, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                         int kb_main, int kb_extra, Sched sched, Epi epi_in, int* status, Comm comm) {
  using L = Gemm2SmemLayout<STAGES, BN2>;
  constexpr int G2_BN = BN2, G2_BNH = BN2 / 2, G2_STAGE_BYTES = L::STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr int CS = EpiColSplit<Epi>::value;
  constexpr int PIPE_THREADS = gemm_pipe_threads<Epi>();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;
  const int my_tiles = sched.tiles_for_cta(cluster_id, n_clusters);
  // a role that gives up raises the flag in both CTAs of the pair: the partner's roles wait on barriers this CTA
  // would have signalled
  const uint32_t partner_abort = mapa_shared(smem_u32(const_cast<const int*>(abort_flag)), rank ^ 1u);
  auto raise_abort = [&]() {
    *abort_flag = 1;
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(partner_abort), "r"(1) : "memory");
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 8 * CS);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc_2cta(tmem_base_slot, TMEM_COLS);
    tmem_relinquish_2cta();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_wait();                  // everything above overlapped the previous kernel's tail (when launched that way)
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if (kb_extra > 0) {
        tma_prefetch_desc(&tmA2);
        tma_prefetch_desc(&tmB2);
      }
      uint32_t it = 0;
      for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
        TileInfo ti = sched.get(cluster_id, n_clusters, t);
        ti.m_blk = ti.m_blk * 2 + static_cast<int>(rank);
        const int row_a = ti.m_blk * GEMM_BM;
        const int row_b = ti.n_blk * G2_BN + static_cast<int>(rank) * G2_BNH + ti.b_row;
        const int nmain = ti.kb_n < 0 ? kb_main : ti.kb_n;
        const int ntile = nmain + (ti.extra ? kb_extra : 0);
        if (!comm.ready(ti)) {
          atomicMax(status, ST_TIMEOUT_PEER);
          raise_abort();
          break;
        }
        for (int kb = 0; kb < ntile; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          // no abort poll in this loop: the time from "stage free" to "loads issued" is on the pipeline's critical
          // path; a partner that gave up is noticed through this wait's own limit
          if (!mbar_wait_abortable(&empty_bar[s], ph ^ 1, abort_flag)) {
            atomicMax(status, ST_TIMEOUT_EMPTY);
            raise_abort();
            break;
          }
          uint8_t* sa = smem + s * G2_STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * G2_STAGE_BYTES);
          const uint32_t fb = mapa_shared(smem_u32(&full_bar[s]), 0);
          if (kb < nmain) {
            tma_load_2d_2cta(sa, &tmA, (ti.kb_lo + kb) * GEMM_BK, row_a, fb);
            tma_load_2d_2cta(sb, &tmB, (ti.kb_lo + kb) * GEMM_BK, row_b, fb);
          } else {
            const int k2 = (kb - nmain) * GEMM_BK;
            tma_load_2d_2cta(sa, &tmA2, k2, row_a, fb);
            tma_load_2d_2cta(sb, &tmB2, k2, row_b, fb);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * GEMM_BM, G2_BN);
      uint32_t it = 0;
      for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
        const int buf = t & 1;
        const uint32_t aph = (t >> 1) & 1;
        if (!mbar_wait_abortable(&tempty_bar[buf], aph ^ 1, abort_flag)) {
          atomicMax(status, ST_TIMEOUT_TMEM_EMPTY);
          raise_abort();
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * G2_BN;
        const TileInfo ti = sched.get(cluster_id, n_clusters, t);
        const int ntile = (ti.kb_n < 0 ? kb_main : ti.kb_n) + (ti.extra ? kb_extra : 0);
        for (int kb = 0; kb < ntile; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_abortable(&full_bar[s], ph, abort_flag)) {
            atomicMax(status, ST_TIMEOUT_FULL);
            raise_abort();
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * G2_STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          const uint64_t adesc = umma_smem_desc_k128(sa);
          const uint64_t bdesc = umma_smem_desc_k128(sb);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k)
            tc_mma_f16_2cta(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
          tc_commit_2cta(&empty_bar[s], 3);   // both CTAs may refill this stage once the MMAs retire
        }
        if (*abort_flag) break;
        tc_commit_2cta(&tfull_bar[buf], 3);   // accumulator complete in both CTAs
      }
    }
  } else if (warp >= 2 + 4 * CS) {
    // ------------------------------------------------------------ communication warps
    comm.push(static_cast<int>(threadIdx.x) - PIPE_THREADS, status);
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    Epi epi = epi_in;
    const int c_begin = epi_col_begin<G2_BN, CS>(), c_end = epi_col_end<G2_BN, CS>();
    const int q = warp & 3;
    const int row = q * 32 + lane;
    for (int t = 0; t < my_tiles; ++t) {
      if (__shfl_sync(0xffffffffu, *abort_flag, 0)) break;
      TileInfo ti = sched.get(cluster_id, n_clusters, t);
      ti.m_blk = ti.m_blk * 2 + static_cast<int>(rank);
      const int buf = t & 1;
      const uint32_t aph = (t >> 1) & 1;
      // per-tile setup (peer-flag waits, first operand prefetches) runs while the tile's MMAs are still in flight
      epi.tile_begin(ti, row);
      const int ok = mbar_wait_abortable(&tfull_bar[buf], aph, abort_flag) ? 1 : 0;
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) {
          atomicMax(status, ST_TIMEOUT_TMEM_FULL);
          raise_abort();
        }
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + buf * G2_BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 32) {
        uint32_t acc[32];
        tmem_ld_32x32(taddr + c, acc);
        tmem_ld_wait();
        epi.chunk(ti, row, c, acc);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tempty_bar[buf]), 0));
      epi.tile_end(ti, row);
    }
    epi_flush(epi, row, 0);
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && !*abort_flag) comm.finish(status);
  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  // neither CTA may leave (or free TMEM) while its partner can still touch its barriers / smem
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc_2cta(tmem_base, TMEM_COLS);
  }
}

}  // namespace artb
