// All-gather -> GEMM in one kernel (column-parallel linear of a tensor-parallel group whose
// activations are sharded along the token dimension).
//
//   C[world*m_seg, N] = gather(X)[world*m_seg, K] * B[N, K]^T (+ gather(T)[.., kt] * B2[N, kt]^T)
//
// Each rank's kernel has four extra warps that push the rank's own shard of X (and of the LoRA
// low-rank activations T) into every peer's copy of the gathered matrix with 16-byte stores over
// NVLink, 32 rows at a time, each followed by a release-store of an arrival flag.  The GEMM tiles
// start with the local segment and move on to the segments of rank+1, rank+2, ...; the TMA
// producer waits (bounded) for the arrival flags of the rows a tile reads.  TMA only reads local
// memory.  The output uses the plain store epilogue (bf16 / fp32 / SwiGLU).
//
// The reference has no tensor parallelism of its own (its `tensor_parallel_size` is a
// pass-through to the inference library, src/art/dev/engine.py:27); the unfused equivalent is an
// NCCL all_gather followed by a library GEMM.
#include "gemm_pipeline_2cta.cuh"
#include "host_utils.h"
#include "tp_policies.cuh"

namespace artb {

template <int BN, int STAGES>
static int launch_ag(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2, const CUtensorMap& tB2,
                     int kb_main, int kb_extra, const SchedSegRot& sched, const EpiStore<BN>& epi, const AgComm& comm,
                     int* status, int max_ctas, cudaStream_t stream) {
  using L = GemmSmemLayout<BN, STAGES>;
  static_assert(L::TOTAL + 4 * EpiStore<BN>::COL_SPLIT * 4096 + 64 <= 227 * 1024, "shared memory");
  auto kern = gemm_tcgen05_kernel<BN, STAGES, SchedSegRot, EpiStore<BN>, AgComm>;
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
  kern<<<grid, gemm_pipe_threads<EpiStore<BN>>() + AgComm::THREADS, L::TOTAL, stream>>>(tA, tB, tA2, tB2, kb_main, kb_extra, sched, epi,
                                                                   status, comm);
  return static_cast<int>(cudaGetLastError());
}

// CTA-pair form (256 x 256 tiles, tcgen05.mma.cta_group::2): used when every rank's token segment is a multiple of
// 256 rows.  Each CTA of a pair waits for, loads and stores its own 128 rows, so the policies are the same objects.
static int launch_ag_pair(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tA2, const CUtensorMap& tB2,
                          int kb_main, int kb_extra, const SchedSegRot& sched, const EpiStore<256>& epi, const AgComm& comm,
                          int* status, int max_ctas, cudaStream_t stream) {
  using L = Gemm2SmemLayout<6, 256>;
  auto kern = gemm_tcgen05_2cta_kernel<6, 256, SchedSegRot, EpiStore<256>, AgComm>;
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
  kern<<<2 * clusters, gemm_pipe_threads<EpiStore<256>>() + AgComm::THREADS, L::TOTAL, stream>>>(tA, tB, tA2, tB2, kb_main, kb_extra, sched,
                                                                          epi, status, comm);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace artb

using namespace artb;

// h            symmetric buffer handle (artb_symm_create); offsets are bytes into its data area,
//              identical on every rank: off_x gathered X [world*m_seg, K] bf16 dense, off_t gathered
//              T [world*m_seg, kt] bf16 dense (kt == 0: none), off_flag uint32 [world][m_seg/32],
//              off_done uint32 [world]
// B, B2        local weight shard [N, K] and scaled LoRA B [N, kt]
// epoch        call number of this (off_x, off_flag) region, starting at 1, same on every rank
// cta_counter  device uint32, zero before the first call
ARTB_EXPORT int artb_tp_ag_gemm(void* h, long off_x, long off_t, int kt, long off_flag, long off_done, const void* B,
                                int ldb, const void* B2, int ldb2, void* C, int ldc, void* H, int ldh,
                                const float* bias, int m_seg, int N, int K, int epilogue, unsigned int epoch,
                                int wait_ms, unsigned int* cta_counter, int* status, int max_ctas,
                                cudaStream_t stream) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || s->world > TP_MAX) return ERR_BAD_SHAPE;
  if (m_seg <= 0 || (m_seg % GEMM_BM) || N <= 0 || (N & 7) || K <= 0 || (K & 7) || (kt & 63)) return ERR_BAD_SHAPE;
  if (epilogue == EPI_BF16_RESID) return ERR_BAD_SHAPE;
  if ((epilogue == EPI_SWIGLU || epilogue == EPI_SWIGLU_BWD) && (!H || (ldh & 7) || (N & 31))) return ERR_BAD_ALIGN;
  if (epilogue != EPI_SWIGLU && epilogue != EPI_SWIGLU_BWD) H = nullptr;
  if ((off_x & 127) || (off_t & 127) || (off_flag & 15) || (off_done & 15)) return ERR_BAD_ALIGN;
  const int world = s->world, M = world * m_seg;
  const int bn = (N >= 256) ? 256 : 128;
  const bool pair = bn == 256 && m_seg % (2 * GEMM_BM) == 0 && max_ctas != 1;
  const int b_box = pair ? 128 : bn;      // a CTA of a pair stages half of the B tile
  char* local = static_cast<char*>(s->table.base[s->rank]);
  CUtensorMap tA, tB, tA2, tB2;
  int e;
  if ((e = make_tmap_bf16_2d(&tA, local + off_x, M, K, K, GEMM_BM, GEMM_BK))) return e;
  if ((e = make_tmap_bf16_2d(&tB, B, N, K, ldb, b_box, GEMM_BK))) return e;
  if (kt > 0) {
    if ((e = make_tmap_bf16_2d(&tA2, local + off_t, M, kt, kt, GEMM_BM, GEMM_BK))) return e;
    if ((e = make_tmap_bf16_2d(&tB2, B2, N, kt, ldb2, b_box, GEMM_BK))) return e;
  } else {
    tA2 = tA;
    tB2 = tB;
  }
  AgComm comm;
  for (int p = 0; p < TP_MAX; ++p) comm.pt.base[p] = p < world ? static_cast<char*>(s->table.base[p]) : nullptr;
  comm.off_x = off_x;
  comm.off_t = off_t;
  comm.off_flag = off_flag;
  comm.off_done = off_done;
  comm.rank = s->rank;
  comm.world = world;
  comm.m_seg = m_seg;
  comm.row_bytes_x = K * 2;
  comm.row_bytes_t = kt * 2;
  comm.epoch = epoch;
  comm.spin = static_cast<uint32_t>(wait_ms <= 0 ? 2000000 : static_cast<long>(wait_ms) * 1000);
  comm.cta_counter = cta_counter;
  const int kb_main = (K + GEMM_BK - 1) / GEMM_BK, kb_extra = kt / GEMM_BK;
  const int bwd = epilogue == EPI_SWIGLU_BWD ? 1 : 0;
  if (pair) {
    SchedSegRot sched{m_seg / (2 * GEMM_BM), (N + 255) / 256, world, s->rank, 0,
                      pick_group_m(m_seg / (2 * GEMM_BM), 2 * GEMM_BM, K)};
    EpiStore<256> epi{C, nullptr, reinterpret_cast<__nv_bfloat16*>(H), bias, ldc, 0, ldh, M, N,
                      epilogue == EPI_F32 ? 1 : 0, N, bwd};
    return launch_ag_pair(tA, tB, tA2, tB2, kb_main, kb_extra, sched, epi, comm, status, max_ctas, stream);
  }
#define ARTB_LAUNCH(BN_, ST_)                                                                                     \
  {                                                                                                               \
    SchedSegRot sched{m_seg / GEMM_BM, (N + BN_ - 1) / BN_, world, s->rank, 0,                                  \
                      pick_group_m(m_seg / GEMM_BM, GEMM_BM, K)};                                   \
    EpiStore<BN_> epi{C, nullptr, reinterpret_cast<__nv_bfloat16*>(H), bias, ldc, 0, ldh, M, N,                   \
                      epilogue == EPI_F32 ? 1 : 0, N, bwd};                                                       \
    return launch_ag<BN_, ST_>(tA, tB, tA2, tB2, kb_main, kb_extra, sched, epi, comm, status, max_ctas, stream);  \
  }
  if (bn == 256) ARTB_LAUNCH(256, 4)
  ARTB_LAUNCH(128, 6)
#undef ARTB_LAUNCH
}
