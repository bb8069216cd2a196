// Expert-parallel combine: the expert owner pushes every output row back to the rank (and row)
// it was dispatched from; the token owner then finishes the receive.
//
//   return   one CTA per row of the owner's expert-ordered buffer: finds the source rank and the
//            row's index in that rank's own sorted order from the exchanged counts, stores the row
//            into the source's return staging buffer over NVLink; the last CTA publishes one
//            arrival flag per peer
//   finish   one CTA per locally sorted row at the token owner: waits (bounded) for the flag of
//            the row's expert owner, copies the row into the caller's private buffer (kept for the
//            backward pass and read by the weighted combine kernel), zero-fills padding rows, and
//            the last CTA tells every peer that the staging buffer may be reused
//
// The weighted sum over a token's k experts is the single-GPU combine kernel (kernels/moe.cu),
// which gathers in a fixed slot order, so the result does not depend on arrival order.
//
// The reference has no expert parallelism.  Unfused equivalent: all_to_all_single + index_add_.
#include <cuda_bf16.h>

#include "ep_layout.cuh"
#include "host_utils.h"
#include "ptx_sm100.cuh"

namespace artb {

__global__ void __launch_bounds__(128)
ep_return_kernel(EpPeers pt, long off_ret, long off_rflag, long off_rdone, int rank, int P, int El,
                 const __nv_bfloat16* __restrict__ yp, int ldy, int D, EpPlan plan, int cap_src, uint32_t epoch,
                 uint32_t spin, int* status, unsigned int* cta_counter) {
  const int R = blockIdx.x;
  __shared__ int s_ok;
  if (R < plan.seg_off[El]) {
    const int j = plan.tile_expert[R >> 7];
    const int o = R - plan.seg_off[j];
    if (o < plan.real_rows[j]) {
      int s = P - 1;
      while (s > 0 && plan.src_start[j * P + s] > o) --s;
      const int dest = plan.src_seg_off[s * El + j] + (o - plan.src_start[j * P + s]);
      if (threadIdx.x == 0) {
        int ok = 1;
        if (epoch > 2)
          ok = wait_flag_ge(reinterpret_cast<const uint32_t*>(ep_base(pt, rank) + off_rdone) + s, epoch - 2, spin);
        if (!ok) atomicMax(status, ST_TIMEOUT_PEER);
        if (dest >= cap_src) {
          atomicMax(status, ST_OVERFLOW);
          ok = 0;
        }
        s_ok = ok;
      }
      __syncthreads();
      if (s_ok) {
        const int nv = D >> 3;
        uint4* dst = reinterpret_cast<uint4*>(ep_base(pt, s) + off_ret) + static_cast<size_t>(dest) * nv;
        const uint4* src = reinterpret_cast<const uint4*>(yp + static_cast<size_t>(R) * ldy);
        for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = src[i];
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(cta_counter, 1u);
    if (prev + 1 == gridDim.x) {
      *cta_counter = 0;
      __threadfence_system();
      for (int p = 0; p < P; ++p) st_release_sys_u32(reinterpret_cast<uint32_t*>(pt.base[p] + off_rflag) + rank, epoch);
    }
  }
}

__global__ void __launch_bounds__(128)
ep_ret_finish_kernel(EpPeers pt, long off_ret, long off_rflag, long off_rdone, int rank, int P, int E, int D,
                     const int* __restrict__ row_token, const int* __restrict__ seg_off_src,
                     const int* __restrict__ tile_expert_src, const int* __restrict__ send_off, int cap_recv,
                     __nv_bfloat16* __restrict__ out, int ldo, uint32_t epoch, uint32_t spin, int* status,
                     unsigned int* cta_counter) {
  const int r = blockIdx.x;
  const int El = E / P;
  __shared__ int s_ok;
  if (r < seg_off_src[E]) {
    const int nv = D >> 3;
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * ldo);
    const int e_r = tile_expert_src[r >> 7];
    // padding rows, and rows the dispatch dropped because their owner was over capacity, come back as zeros
    if (row_token[r] < 0 || send_off[e_r] + (r - seg_off_src[e_r]) >= cap_recv) {
      for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    } else {
      const int owner = e_r / El;
      if (threadIdx.x == 0) {
        const int ok = wait_flag_ge(reinterpret_cast<const uint32_t*>(pt.base[rank] + off_rflag) + owner, epoch, spin);
        if (!ok) atomicMax(status, ST_TIMEOUT_PEER);
        s_ok = ok;
      }
      __syncthreads();
      if (s_ok) {
        const uint4* src = reinterpret_cast<const uint4*>(pt.base[rank] + off_ret) + static_cast<size_t>(r) * nv;
        for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = __ldcg(src + i);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(cta_counter, 1u);
    if (prev + 1 == gridDim.x) {
      *cta_counter = 0;
      __threadfence_system();
      for (int p = 0; p < P; ++p) st_release_sys_u32(reinterpret_cast<uint32_t*>(pt.base[p] + off_rdone) + rank, epoch);
    }
  }
}

static void fill_peers(EpPeers& pt, const SymmState* s) {
  for (int p = 0; p < EP_MAX_RANKS; ++p) pt.base[p] = p < s->world ? static_cast<char*>(s->table.base[p]) : nullptr;
}

static uint32_t spin_for(int wait_ms) {
  return static_cast<uint32_t>(wait_ms <= 0 ? 2000000 : static_cast<long>(wait_ms) * 1000);
}

}  // namespace artb

using namespace artb;

// yp bf16 [cap_recv, D] private (expert order of this rank); rows go back to their sources.
ARTB_EXPORT int artb_ep_return(void* h, long off_ret, long off_rflag, long off_rdone, int E, const void* yp, int ldy,
                               int D, int** plan_ptrs, int cap_recv, int cap_src, unsigned int epoch, int wait_ms,
                               int* status, unsigned int* cta_counter, cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || (D & 7) || (ldy & 7) || cap_recv <= 0) return ERR_BAD_SHAPE;
  EpPeers pt;
  fill_peers(pt, s);
  EpPlan plan{plan_ptrs[0], plan_ptrs[1], plan_ptrs[2], plan_ptrs[3], plan_ptrs[4], plan_ptrs[5], plan_ptrs[6]};
  ep_return_kernel<<<cap_recv, 128, 0, st>>>(pt, off_ret, off_rflag, off_rdone, s->rank, s->world, E / s->world,
                                             reinterpret_cast<const __nv_bfloat16*>(yp), ldy, D, plan, cap_src, epoch,
                                             spin_for(wait_ms), status, cta_counter);
  return static_cast<int>(cudaGetLastError());
}

// out bf16 [cap_src, D] private, in this rank's own expert-sorted row order.
ARTB_EXPORT int artb_ep_ret_finish(void* h, long off_ret, long off_rflag, long off_rdone, int E, int D,
                                   const int* row_token, const int* seg_off_src, const int* tile_expert_src,
                                   const int* send_off, int cap_recv, void* out, int ldo, int cap_src, unsigned int epoch,
                                   int wait_ms, int* status, unsigned int* cta_counter, cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || (D & 7) || (ldo & 7) || cap_src <= 0) return ERR_BAD_SHAPE;
  EpPeers pt;
  fill_peers(pt, s);
  ep_ret_finish_kernel<<<cap_src, 128, 0, st>>>(pt, off_ret, off_rflag, off_rdone, s->rank, s->world, E, D, row_token,
                                                seg_off_src, tile_expert_src, send_off, cap_recv,
                                                reinterpret_cast<__nv_bfloat16*>(out), ldo, epoch, spin_for(wait_ms), status,
                                                cta_counter);
  return static_cast<int>(cudaGetLastError());
}
