// Warp-specialised, persistent tcgen05 GEMM pipeline for sm_100a.
//
//   D[128 x BN] (fp32, TMEM) = A[128 x K] * B[BN x K]^T      (both operands K-major bf16)
//
// One CTA = 6 or 10 warps (+ communication warps of a fused collective):
//   warp 0      TMA producer  (one elected lane issues cp.async.bulk.tensor loads)
//   warp 1      MMA issuer    (one elected lane issues tcgen05.mma; the warp owns TMEM alloc/dealloc)
//   warps 2..5  epilogue      (each reads its 32-lane quarter of TMEM with tcgen05.ld)
//   warps 6..9  second epilogue set, when the epilogue policy asks for it (COL_SPLIT = 2): the two warps of a lane
//               quarter then take half of the tile's columns each.  One warp per scheduler issues an instruction
//               every ~8 cycles (dependent fixed-latency arithmetic); an epilogue with real arithmetic in it (SwiGLU
//               backward: ~40 instructions per element) is then slower than the tile's main loop, two warps are not.
//
// The accumulator is double-buffered in TMEM (2 x BN columns) so the epilogue of
// tile i overlaps the main loop of tile i+1.  Operand stages live in shared
// memory in the 128-byte-swizzled layout that TMA writes and UMMA reads.
//
// An optional second operand pair (A2, B2) is appended along K ("extra-K"): the
// low-rank LoRA update  T[M x r] * (s*Bl)[N x r]^T  is accumulated by the tensor
// cores into the same TMEM tile as the frozen-weight product, at the cost of one
// extra 64-wide K block.
//
// Scheduling (which tiles a CTA visits, in which order) and the epilogue (what
// happens to each 32-column slab of the accumulator) are template policies, so
// the plain GEMM, the residual/SwiGLU variants and the fused LM-head log-prob
// kernel share this file.
#pragma once
#include "ptx_sm100.cuh"

namespace artb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;   // pipeline threads of a kernel whose epilogue policy does not split columns

// Epilogue policies may declare `static constexpr int COL_SPLIT = 2` (default 1).
template <class E, class = void>
struct EpiColSplit {
  static constexpr int value = 1;
};
template <class E>
struct EpiColSplit<E, decltype(void(E::COL_SPLIT))> {
  static constexpr int value = E::COL_SPLIT;
};
// threads of the producer, MMA and epilogue warps (communication warps come after them)
template <class Epi>
constexpr int gemm_pipe_threads() {
  return 64 + 128 * EpiColSplit<Epi>::value;
}
// Index of the calling epilogue warp (0 .. 4 * COL_SPLIT - 1) and the column range [begin, end) of a BN-wide tile it
// handles (multiples of 32; with an odd number of chunks the first set takes one more).
__device__ __forceinline__ int epi_warp_slot() { return static_cast<int>(threadIdx.x >> 5) - 2; }
template <int BN, int CS>
__device__ __forceinline__ int epi_col_begin() {
  return CS == 1 ? 0 : (epi_warp_slot() >> 2) * (((BN / 32 + 1) / 2) * 32);
}
template <int BN, int CS>
__device__ __forceinline__ int epi_col_end() {
  return (CS == 1 || (epi_warp_slot() >> 2) == 1) ? BN : ((BN / 32 + 1) / 2) * 32;
}

struct TileInfo {
  int m_blk;   // tile row index   (rows m_blk*128 ..)
  int n_blk;   // tile column index (cols n_blk*BN ..)
  int first;   // first tile of an epilogue group (policy-defined)
  int last;    // last tile of an epilogue group
  int group;   // policy-defined group id (e.g. vocabulary split, K split)
  int kb_lo;   // first main-operand K block of this tile (split-K); 0 for a full tile
  int kb_n;    // number of main-operand K blocks; < 0 means "all of them"
  int extra;   // include the extra-K operand blocks in this tile
  int b_row;   // row offset added to the B / B2 coordinates (grouped GEMM: expert * rows per expert)
};

__device__ __forceinline__ TileInfo make_tile(int m_blk, int n_blk) {
  TileInfo ti;
  ti.m_blk = m_blk;
  ti.n_blk = n_blk;
  ti.first = ti.last = 1;
  ti.group = 0;
  ti.kb_lo = 0;
  ti.kb_n = -1;
  ti.extra = 1;
  ti.b_row = 0;
  return ti;
}

// Grouped tile order: the M tiles are cut into bands of `group_m`; inside a band M runs fastest, then N; the bands
// follow one another.  The CTAs that run at the same time then share a band of A (group_m * tile rows * K, sized by the
// host to stay resident in L2) while B streams through once per band, instead of sweeping all of A for every few
// columns of B.
__device__ __forceinline__ void raster_tile(int tile, int m_tiles, int n_tiles, int group_m, int& m, int& n) {
  const int per_group = group_m * n_tiles;
  const int g = tile / per_group, r = tile - g * per_group;
  const int rows = min(group_m, m_tiles - g * group_m);
  m = g * group_m + r % rows;
  n = r / rows;
}

template <int BN, int STAGES>
struct GemmSmemLayout {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // full[STAGES] empty[STAGES] tmem_full[2] tmem_empty[2] | tmem_base | abort
  static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
  static constexpr int TOTAL = BAR_OFFSET + BAR_BYTES + 1024;  // + alignment slack
};

// Communication policy of a fused compute+collective kernel.  `THREADS` extra threads (whole
// warps, after the six pipeline warps) run `push()` concurrently with the main loop; the producer
// calls `ready()` before the first load of a tile (bounded wait on data pushed by peers); thread 0
// calls `finish()` after every store of the CTA has been issued.
struct NoComm {
  static constexpr int THREADS = 0;
  __device__ void push(int /*tid*/, int* /*status*/) const {}
  __device__ bool ready(const TileInfo&) const { return true; }
  __device__ void finish(int* /*status*/) const {}
};

// Optional epilogue hook `flush(row)`: called by every epilogue thread after its last tile (policies that defer work,
// e.g. the publication of arrival flags, finish it there).
template <class E>
__device__ __forceinline__ auto epi_flush(E& e, int row, int) -> decltype(e.flush(row), void()) {
  e.flush(row);
}
template <class E>
__device__ __forceinline__ void epi_flush(E&, int, long) {}

template <int BN, int STAGES, class Sched, class Epi, class Comm = NoComm>
__global__ void __launch_bounds__(gemm_pipe_threads<Epi>() + Comm::THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmA2,
                    const __grid_constant__ CUtensorMap tmB2, int kb_main, int kb_extra,
                    Sched sched, Epi epi_in, int* status, Comm comm) {
  using L = GemmSmemLayout<BN, STAGES>;
  // two accumulators of BN columns each; the allocation is rounded up to a power of two
  constexpr uint32_t TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
  static_assert(BN % 32 == 0 && BN <= 256, "BN");
  constexpr int CS = EpiColSplit<Epi>::value;
  constexpr int PIPE_THREADS = gemm_pipe_threads<Epi>();
  static_assert(CS == 1 || (CS == 2 && BN >= 64), "COL_SPLIT");

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
  const int my_tiles = sched.tiles_for_cta(blockIdx.x, gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 4 * CS);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_wait();                  // everything above overlapped the previous kernel's tail (when launched that way)
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      if (kb_extra > 0) {
        tma_prefetch_desc(&tmA2);
        tma_prefetch_desc(&tmB2);
      }
      uint32_t it = 0;
      for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
        const TileInfo ti = sched.get(blockIdx.x, gridDim.x, t);
        const int nmain = ti.kb_n < 0 ? kb_main : ti.kb_n;
        const int ntile = nmain + (ti.extra ? kb_extra : 0);
        if (!comm.ready(ti)) {
          atomicMax(status, ST_TIMEOUT_PEER);
          *abort_flag = 1;
          break;
        }
        for (int kb = 0; kb < ntile; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_abortable(&empty_bar[s], ph ^ 1, abort_flag)) {
            atomicMax(status, ST_TIMEOUT_EMPTY);
            *abort_flag = 1;
            break;
          }
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
          if (kb < nmain) {
            tma_load_2d(sa, &tmA, (ti.kb_lo + kb) * GEMM_BK, ti.m_blk * GEMM_BM, &full_bar[s]);
            tma_load_2d(sb, &tmB, (ti.kb_lo + kb) * GEMM_BK, ti.n_blk * BN + ti.b_row, &full_bar[s]);
          } else {
            const int k2 = (kb - nmain) * GEMM_BK;
            tma_load_2d(sa, &tmA2, k2, ti.m_blk * GEMM_BM, &full_bar[s]);
            tma_load_2d(sb, &tmB2, k2, ti.n_blk * BN + ti.b_row, &full_bar[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(GEMM_BM, BN);
      uint32_t it = 0;
      for (int t = 0; t < my_tiles && !*abort_flag; ++t) {
        const int buf = t & 1;
        const uint32_t aph = (t >> 1) & 1;
        if (!mbar_wait_abortable(&tempty_bar[buf], aph ^ 1, abort_flag)) {
          atomicMax(status, ST_TIMEOUT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        const TileInfo ti = sched.get(blockIdx.x, gridDim.x, t);
        const int ntile = (ti.kb_n < 0 ? kb_main : ti.kb_n) + (ti.extra ? kb_extra : 0);
        for (int kb = 0; kb < ntile; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_abortable(&full_bar[s], ph, abort_flag)) {
            atomicMax(status, ST_TIMEOUT_FULL);
            *abort_flag = 1;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          const uint64_t adesc = umma_smem_desc_k128(sa);
          const uint64_t bdesc = umma_smem_desc_k128(sb);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            // advance 16 bf16 = 32 B along K inside the swizzled row: +2 in 16-byte units
            tc_mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
          }
          tc_commit(&empty_bar[s]);  // stage reusable once these MMAs retire
        }
        if (*abort_flag) break;
        tc_commit(&tfull_bar[buf]);  // accumulator complete
      }
    }
  } else if (warp >= 2 + 4 * CS) {
    // ------------------------------------------------------------ communication warps
    comm.push(static_cast<int>(threadIdx.x) - PIPE_THREADS, status);
  } else {
    // ------------------------------------------------------------ epilogue
    Epi epi = epi_in;
    const int c_begin = epi_col_begin<BN, CS>(), c_end = epi_col_end<BN, CS>();
    const int q = warp & 3;  // TMEM lane quarter this warp may touch
    const int row = q * 32 + lane;
    for (int t = 0; t < my_tiles; ++t) {
      // Abort decisions are made warp-uniform: the TMEM loads below are .sync.aligned.
      if (__shfl_sync(0xffffffffu, *abort_flag, 0)) break;
      const TileInfo ti = sched.get(blockIdx.x, gridDim.x, t);
      const int buf = t & 1;
      const uint32_t aph = (t >> 1) & 1;
      // per-tile setup (peer-flag waits, first operand prefetches) runs while the tile's MMAs are still in flight
      epi.tile_begin(ti, row);
      const int ok = mbar_wait_abortable(&tfull_bar[buf], aph, abort_flag) ? 1 : 0;
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) {
          atomicMax(status, ST_TIMEOUT_TMEM_FULL);
          *abort_flag = 1;
        }
        break;
      }
      tc_fence_after_sync();
      const uint32_t taddr = tmem_base + buf * BN + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = c_begin; c < c_end; c += 32) {
        uint32_t acc[32];
        tmem_ld_32x32(taddr + c, acc);
        tmem_ld_wait();
        epi.chunk(ti, row, c, acc);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[buf]);
      epi.tile_end(ti, row);
    }
    epi_flush(epi, row, 0);
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && !*abort_flag) comm.finish(status);
  if (*abort_flag) {
    // Give any copy that is still in flight time to land before smem is released.
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace artb
