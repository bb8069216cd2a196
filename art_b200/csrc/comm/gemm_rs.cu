// GEMM -> reduce-scatter in one kernel (row-parallel linear of a tensor-parallel group; the output
// is sharded along the token dimension).
//
//   out[m_seg, N] (rank r) = sum_p ( A_p[rows of r, K_p] * B_p[N, K_p]^T + A2_p * B2^T ) + R_r
//
// Each rank computes its partial product for ALL token rows.  Tiles whose rows belong to another
// rank are stored straight from the epilogue registers into that rank's bf16 staging area over
// NVLink (re-laid out through shared memory so that 8 lanes write 128 contiguous bytes; one
// release flag per tile and epilogue warp); the rank's own tiles are
// scheduled last, and their epilogue adds the partials the peers have pushed meanwhile, plus the
// residual shard, and writes the final bf16 rows.  There is no separate reduction kernel, no
// atomics, and the summation order is fixed (deterministic).
//
// Unfused equivalent: a library GEMM followed by an NCCL reduce_scatter.  The reference has no
// tensor parallelism of its own (src/art/dev/engine.py:27 forwards `tensor_parallel_size` to the
// inference library).
#include <string.h>

#include "gemm_pipeline_2cta.cuh"
#include "host_utils.h"
#include "tp_policies.cuh"

namespace artb {

template <int BN, int STAGES>
static int launch_rs(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2, const CUtensorMap& tB2,
                     int kb_main, int kb_extra, const SchedSegRot& sched, const EpiReduceScatter<BN>& epi,
                     const RsComm& comm, int* status, int max_ctas, cudaStream_t stream) {
  using L = GemmSmemLayout<BN, STAGES>;
  static_assert(L::TOTAL + 8 * 4096 + 64 <= 227 * 1024, "shared memory");
  auto kern = gemm_tcgen05_kernel<BN, STAGES, SchedSegRot, EpiReduceScatter<BN>, RsComm>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  int grid = sched.seg_m_tiles * sched.n_tiles * sched.world;
  int cap = sm_count();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  if (grid > cap) grid = cap;
  kern<<<grid, gemm_pipe_threads<EpiReduceScatter<BN>>() + RsComm::THREADS, L::TOTAL, stream>>>(tA, tB, tA2, tB2, kb_main, kb_extra,
                                                                                              sched, epi, status, comm);
  return static_cast<int>(cudaGetLastError());
}

// CTA-pair form (256 x 256 tiles): each CTA of a pair scatters / reduces its own 128 x 256 half of the tile.
static int launch_rs_pair(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2, const CUtensorMap& tB2,
                          int kb_main, int kb_extra, const SchedSegRot& sched, const EpiReduceScatter<256>& epi,
                          const RsComm& comm, int* status, int max_ctas, cudaStream_t stream) {
  using L = Gemm2SmemLayout<6, 256>;
  auto kern = gemm_tcgen05_2cta_kernel<6, 256, SchedSegRot, EpiReduceScatter<256>, RsComm>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured[dev & 63]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev & 63] = true;
  }
  int clusters = sched.seg_m_tiles * sched.n_tiles * sched.world;
  int cap = sm_count() / 2;
  if (max_ctas > 0 && max_ctas / 2 < cap) cap = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (clusters > cap) clusters = cap;
  kern<<<2 * clusters, gemm_pipe_threads<EpiReduceScatter<256>>() + RsComm::THREADS, L::TOTAL, stream>>>(
      tA, tB, tA2, tB2, kb_main, kb_extra, sched, epi, status, comm);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace artb

using namespace artb;

// h            symmetric buffer handle; byte offsets into its data area, identical on every rank:
//              off_stage bf16 [world-1][m_seg][N], off_flag uint32 [world-1][tile_cap][8],
//              off_done uint32 [world]
// A, B         local operands [world*m_seg, K] and [N, K] (K = this rank's slice of the reduction dim)
// A2, B2, K2   optional extra-K pair (LoRA partial), K2 multiple of 8
// out, R       bf16 [m_seg, N] result shard and optional residual shard
// tile_cap     flags per staging slot; >= (m_seg/128) * ceil(N/256)
ARTB_EXPORT int artb_tp_gemm_rs(void* h, long off_stage, long off_flag, long off_done, int tile_cap, const void* A,
                                int lda, const void* B, int ldb, const void* A2, int lda2, const void* B2, int ldb2,
                                int K2, void* out, int ldc, const void* R, int ldr, int m_seg, int N, int K,
                                unsigned int epoch, int wait_ms, unsigned int* cta_counter, int* status, int max_ctas,
                                cudaStream_t stream) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || s->world > TP_MAX) return ERR_BAD_SHAPE;
  if (m_seg <= 0 || (m_seg % GEMM_BM) || N <= 0 || (N & 7) || K <= 0 || (K & 7) || K2 < 0 || (K2 & 7))
    return ERR_BAD_SHAPE;
  if ((off_stage & 127) || (off_flag & 15) || (off_done & 15) || (ldc & 7) || (R && (ldr & 7))) return ERR_BAD_ALIGN;
  const int world = s->world, M = world * m_seg;
  int cap = sm_count();
  if (max_ctas > 0 && max_ctas < cap) cap = max_ctas;
  const int bn = 256;   // EpiReduceScatter pairs 32-column slabs: the tile width must be a multiple of 64
  const int n_tiles = (N + bn - 1) / bn;
  if ((m_seg / GEMM_BM) * n_tiles > tile_cap) return ERR_TOO_LARGE;
  const bool pair = m_seg % (2 * GEMM_BM) == 0 && max_ctas != 1;
  const int b_box = pair ? bn / 2 : bn;      // a CTA of a pair stages half of the B tile
  CUtensorMap tA, tB, tA2, tB2;
  int e;
  if ((e = make_tmap_bf16_2d(&tA, A, M, K, lda, GEMM_BM, GEMM_BK))) return e;
  if ((e = make_tmap_bf16_2d(&tB, B, N, K, ldb, b_box, GEMM_BK))) return e;
  if (K2 > 0) {
    if ((e = make_tmap_bf16_2d(&tA2, A2, M, K2, lda2, GEMM_BM, GEMM_BK))) return e;
    if ((e = make_tmap_bf16_2d(&tB2, B2, N, K2, ldb2, b_box, GEMM_BK))) return e;
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  EpiReduceScatter<256> epi;
  RsComm comm;
  for (int p = 0; p < TP_MAX; ++p) {
    epi.pt.base[p] = p < world ? static_cast<char*>(s->table.base[p]) : nullptr;
    comm.pt.base[p] = epi.pt.base[p];
  }
  epi.off_stage = off_stage;
  epi.off_flag = off_flag;
  epi.off_done = off_done;
  epi.out = reinterpret_cast<__nv_bfloat16*>(out);
  epi.R = reinterpret_cast<const __nv_bfloat16*>(R);
  epi.ldc = ldc;
  epi.ldr = ldr;
  epi.N = N;
  epi.m_seg = m_seg;
  epi.n_tiles = n_tiles;
  epi.tile_cap = tile_cap;
  epi.rank = s->rank;
  epi.world = world;
  epi.epoch = epoch;
  epi.spin = static_cast<uint32_t>(wait_ms <= 0 ? 2000000 : static_cast<long>(wait_ms) * 1000);
  epi.status = status;
  epi.own = 0;
  epi.pre_ok = 0;
  epi.done_seen = 0;
  epi.lrow = 0;
  epi.stage = nullptr;
  epi.flag = nullptr;
  comm.off_done = off_done;
  comm.rank = s->rank;
  comm.world = world;
  comm.epoch = epoch;
  comm.cta_counter = cta_counter;
  SchedSegRot sched{m_seg / GEMM_BM, n_tiles, world, s->rank, 1, pick_group_m(m_seg / GEMM_BM, GEMM_BM, K)};
  const int kb_main = (K + GEMM_BK - 1) / GEMM_BK, kb_extra = (K2 + GEMM_BK - 1) / GEMM_BK;
  if (pair) {
    int cl = sm_count() / 2;
    if (max_ctas > 0 && max_ctas / 2 < cl) cl = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
    SchedSegRot sched2{m_seg / (2 * GEMM_BM), n_tiles, world, s->rank, 1, pick_group_m(m_seg / (2 * GEMM_BM), 2 * GEMM_BM, K),
                       2 * cl};      // own tiles two grid waves behind the peers' tiles
    return launch_rs_pair(tA, tB, tA2, tB2, kb_main, kb_extra, sched2, epi, comm, status, max_ctas, stream);
  }
  return launch_rs<256, 4>(tA, tB, tA2, tB2, kb_main, kb_extra, sched, epi, comm, status, max_ctas, stream);
}
