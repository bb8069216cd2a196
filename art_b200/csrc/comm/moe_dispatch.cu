// Expert-parallel dispatch: count exchange, row push to the expert owners, receive-side finish.
//
//   exchange  all-gather of the per-expert token counts (P x E int32) through peer stores + epoch
//             flags, then every rank derives all offsets of the call (see ep_layout.cuh)
//   dispatch  one CTA per locally sorted row: x[token] (optionally times its routing weight) is
//             stored into the owner's receive staging buffer over NVLink; the CTA that completes an
//             expert's rows publishes the (expert, source) arrival flag
//   recv      one CTA per staged row at the owner: waits (bounded) for the arrival flags of the
//             row's expert, copies the row into the caller's private activation buffer (which the
//             grouped GEMMs and the backward pass read), zero-fills the 128-row padding, and the
//             last CTA tells every peer that the staging buffer may be reused
//
// Plain ld/st over peer pointers only; every wait is bounded (ST_TIMEOUT_PEER); a receive buffer
// that is too small for the routing at hand reports ST_OVERFLOW instead of writing out of range.
//
// The reference has no expert parallelism (dense models only).  Unfused equivalent:
// torch.distributed.all_to_all_single of counts, then of the permuted rows.
#include <cuda_bf16.h>

#include "ep_layout.cuh"
#include "host_utils.h"
#include "ptx_sm100.cuh"

namespace artb {

__global__ void __launch_bounds__(256)
ep_exchange_kernel(EpPeers pt, long off_cnt, long off_cnt_flag, int rank, int P, int E, const int* __restrict__ counts,
                   uint32_t epoch, uint32_t spin, EpPlan plan, int cap_tiles, int* status) {
  __shared__ int s_ok;
  __shared__ int s_seg[EP_MAX_EXPERTS + 1];
  const int tid = threadIdx.x;
  const int El = E / P;
  if (tid == 0) s_ok = 1;
  for (int p = 0; p < P; ++p) {
    int* dst = reinterpret_cast<int*>(pt.base[p] + off_cnt) + rank * E;
    for (int e = tid; e < E; e += blockDim.x) dst[e] = counts[e];
  }
  __threadfence_system();
  __syncthreads();
  if (tid < P) {
    st_release_sys_u32(reinterpret_cast<uint32_t*>(pt.base[tid] + off_cnt_flag) + rank, epoch);
    if (!wait_flag_ge(reinterpret_cast<const uint32_t*>(pt.base[rank] + off_cnt_flag) + tid, epoch, spin)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) {
    if (tid == 0) atomicMax(status, ST_TIMEOUT_PEER);
    return;
  }
  const int* cnt = reinterpret_cast<const int*>(pt.base[rank] + off_cnt);
  for (int i = tid; i < P * E; i += blockDim.x) plan.cnt_all[i] = __ldcg(cnt + i);
  __syncthreads();
  const int* ca = plan.cnt_all;
  for (int e = tid; e < E; e += blockDim.x) {
    const int owner = e / El, j = e - owner * El;
    int seg = 0;   // start of expert e's segment in its owner's receive order
    for (int j2 = 0; j2 < j; ++j2) {
      int tot = 0;
      for (int s = 0; s < P; ++s) tot += ca[s * E + owner * El + j2];
      seg += (tot + 127) / 128 * 128;
    }
    int before = 0, tot = 0;
    for (int s = 0; s < P; ++s) {
      if (s < rank) before += ca[s * E + e];
      tot += ca[s * E + e];
    }
    plan.send_off[e] = seg + before;
    if (owner == rank) {
      // Everything the owner indexes is clipped to the receive capacity: rows that would land beyond it are dropped
      // by their senders (same arithmetic on every rank), their segments shrink or become empty here.
      const int cap_rows = cap_tiles * 128;
      const int seg_c = seg < cap_rows ? seg : cap_rows;
      const int end_c = seg + (tot + 127) / 128 * 128 < cap_rows ? seg + (tot + 127) / 128 * 128 : cap_rows;
      s_seg[j] = seg_c;
      plan.real_rows[j] = tot < cap_rows - seg_c ? tot : cap_rows - seg_c;
      if (j == El - 1) s_seg[El] = end_c > seg_c ? end_c : seg_c;
      int run = 0;
      for (int s = 0; s < P; ++s) {
        plan.src_start[j * P + s] = run;
        run += ca[s * E + e];
        int off = 0;   // source s's own sorted order: segments of ALL experts, each padded to 128
        for (int e2 = 0; e2 < e; ++e2) off += (ca[s * E + e2] + 127) / 128 * 128;
        plan.src_seg_off[s * El + j] = off;
      }
    }
  }
  __syncthreads();
  for (int j = tid; j <= El; j += blockDim.x) plan.seg_off[j] = s_seg[j];
  for (int t = tid; t < cap_tiles; t += blockDim.x) {
    const int row = t * 128;
    int ex = -1;
    if (row < s_seg[El]) {
      int lo = 0, hi = El;
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_seg[mid] <= row) lo = mid;
        else hi = mid;
      }
      ex = lo;
    }
    plan.tile_expert[t] = ex;
  }
}

__device__ __forceinline__ void ep_copy_row(uint4* dst, const uint4* src, int nv, float w, bool use_w) {
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    uint4 v = src[i];
    if (use_w) {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        h[j] = __floats2bfloat162_rn(f.x * w, f.y * w);
      }
    }
    dst[i] = v;
  }
}

__global__ void __launch_bounds__(128)
ep_dispatch_kernel(EpPeers pt, long off_recv, long off_dflag, long off_ddone, int rank, int P, int E,
                   const __nv_bfloat16* __restrict__ x, int ldx, int D, const int* __restrict__ row_token,
                   const float* __restrict__ row_w, int use_w, const int* __restrict__ seg_off_src,
                   const int* __restrict__ tile_expert_src, EpPlan plan, int cap_recv, int* __restrict__ done_cnt,
                   uint32_t epoch, uint32_t spin, int allow_drop, int* status) {
  const int El = E / P;
  const int r = blockIdx.x;
  if (r == static_cast<int>(gridDim.x) - 1) {
    // experts this rank sends nothing to still need their arrival flag
    for (int e = threadIdx.x; e < E; e += blockDim.x)
      if (plan.cnt_all[rank * E + e] == 0) {
        const int owner = e / El, j = e - owner * El;
        st_release_sys_u32(reinterpret_cast<uint32_t*>(ep_base(pt, owner) + off_dflag) + j * P + rank, epoch);
      }
    return;
  }
  if (r >= seg_off_src[E]) return;
  const int t = row_token[r];
  if (t < 0) return;
  const int e = tile_expert_src[r >> 7];
  const int owner = e / El, j = e - owner * El;
  const int dest = plan.send_off[e] + (r - seg_off_src[e]);
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    if (epoch > 2)   // the owner has consumed the call that last used this parity of its staging buffer
      ok = wait_flag_ge(reinterpret_cast<const uint32_t*>(ep_base(pt, rank) + off_ddone) + owner, epoch - 2, spin);
    if (!ok) atomicMax(status, ST_TIMEOUT_PEER);
    if (dest >= cap_recv) {
      // beyond the owner's capacity: the row is dropped (it contributes zero; status[1] counts such rows); unless the
      // caller allows dropping this is an error
      atomicAdd(status + 1, 1);
      if (!allow_drop) atomicMax(status, ST_OVERFLOW);
      ok = 0;
    }
    s_ok = ok;
  }
  __syncthreads();
  if (s_ok) {
    uint4* dst = reinterpret_cast<uint4*>(ep_base(pt, owner) + off_recv) + static_cast<size_t>(dest) * (D >> 3);
    ep_copy_row(dst, reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * ldx), D >> 3, use_w ? row_w[r] : 1.f,
                use_w != 0);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int c = atomicAdd(done_cnt + e, 1) + 1;
    if (c == plan.cnt_all[rank * E + e]) {
      done_cnt[e] = 0;
      __threadfence();
      st_release_sys_u32(reinterpret_cast<uint32_t*>(ep_base(pt, owner) + off_dflag) + j * P + rank, epoch);
    }
  }
}

// Publishes `epoch` into slot [rank] of the done words of every peer once the last CTA retires.
__device__ __forceinline__ void ep_publish_last(const EpPeers& pt, long off_done, int rank, int P, uint32_t epoch,
                                                unsigned int* cta_counter) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int prev = atomicAdd(cta_counter, 1u);
    if (prev + 1 == gridDim.x) {
      *cta_counter = 0;
      __threadfence_system();
      for (int p = 0; p < P; ++p) st_release_sys_u32(reinterpret_cast<uint32_t*>(pt.base[p] + off_done) + rank, epoch);
    }
  }
}

__global__ void __launch_bounds__(128)
ep_recv_kernel(EpPeers pt, long off_recv, long off_dflag, long off_ddone, int rank, int P, int El, int D, EpPlan plan,
               __nv_bfloat16* __restrict__ out, int ldo, uint32_t epoch, uint32_t spin, int* status,
               unsigned int* cta_counter) {
  const int R = blockIdx.x;
  __shared__ int s_ok;
  if (R < plan.seg_off[El]) {
    const int j = plan.tile_expert[R >> 7];
    const int o = R - plan.seg_off[j];
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(R) * ldo);
    const int nv = D >> 3;
    if (o >= plan.real_rows[j]) {
      for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    } else {
      if (threadIdx.x == 0) {
        int ok = 1;
        const uint32_t* fl = reinterpret_cast<const uint32_t*>(pt.base[rank] + off_dflag) + j * P;
        for (int s = 0; s < P; ++s)
          if (!wait_flag_ge(fl + s, epoch, spin)) ok = 0;
        if (!ok) atomicMax(status, ST_TIMEOUT_PEER);
        s_ok = ok;
      }
      __syncthreads();
      if (s_ok) {
        const uint4* src = reinterpret_cast<const uint4*>(pt.base[rank] + off_recv) + static_cast<size_t>(R) * nv;
        for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = __ldcg(src + i);
      }
    }
  }
  ep_publish_last(pt, off_ddone, rank, P, epoch, cta_counter);
}

static void fill_peers(EpPeers& pt, const SymmState* s) {
  for (int p = 0; p < EP_MAX_RANKS; ++p) pt.base[p] = p < s->world ? static_cast<char*>(s->table.base[p]) : nullptr;
}

static uint32_t spin_for(int wait_ms) {
  return static_cast<uint32_t>(wait_ms <= 0 ? 2000000 : static_cast<long>(wait_ms) * 1000);
}

}  // namespace artb

using namespace artb;

// plan_ptrs: the seven device int32 arrays of EpPlan, in declaration order.
ARTB_EXPORT int artb_ep_exchange(void* h, long off_cnt, long off_cnt_flag, int E, const int* counts, unsigned int epoch,
                                 int wait_ms, int** plan_ptrs, int cap_tiles, int* status, cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || s->world > EP_MAX_RANKS || E <= 0 || E > EP_MAX_EXPERTS || E % s->world) return ERR_BAD_SHAPE;
  EpPeers pt;
  fill_peers(pt, s);
  EpPlan plan{plan_ptrs[0], plan_ptrs[1], plan_ptrs[2], plan_ptrs[3], plan_ptrs[4], plan_ptrs[5], plan_ptrs[6]};
  ep_exchange_kernel<<<1, 256, 0, st>>>(pt, off_cnt, off_cnt_flag, s->rank, s->world, E, counts, epoch,
                                        spin_for(wait_ms), plan, cap_tiles, status);
  return static_cast<int>(cudaGetLastError());
}

// x bf16 [M, D] (ldx); row_token / row_w / seg_off_src / tile_expert_src: the local expert-sorted plan
// (cap_src rows).  done_cnt: device int32 [E], zero before the first call.
ARTB_EXPORT int artb_ep_dispatch(void* h, long off_recv, long off_dflag, long off_ddone, int E, const void* x, int ldx,
                                 int D, const int* row_token, const float* row_w, int use_w, const int* seg_off_src,
                                 const int* tile_expert_src, int cap_src, int** plan_ptrs, int cap_recv, int* done_cnt,
                                 unsigned int epoch, int wait_ms, int allow_drop, int* status, cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || (D & 7) || (ldx & 7) || cap_src <= 0) return ERR_BAD_SHAPE;
  EpPeers pt;
  fill_peers(pt, s);
  EpPlan plan{plan_ptrs[0], plan_ptrs[1], plan_ptrs[2], plan_ptrs[3], plan_ptrs[4], plan_ptrs[5], plan_ptrs[6]};
  ep_dispatch_kernel<<<cap_src + 1, 128, 0, st>>>(pt, off_recv, off_dflag, off_ddone, s->rank, s->world, E,
                                                  reinterpret_cast<const __nv_bfloat16*>(x), ldx, D, row_token, row_w,
                                                  use_w, seg_off_src, tile_expert_src, plan, cap_recv, done_cnt, epoch,
                                                  spin_for(wait_ms), allow_drop, status);
  return static_cast<int>(cudaGetLastError());
}

// out bf16 [cap_recv, D] private; cta_counter device uint32, zero before the first call.
ARTB_EXPORT int artb_ep_recv(void* h, long off_recv, long off_dflag, long off_ddone, int E, int D, int** plan_ptrs,
                             void* out, int ldo, int cap_recv, unsigned int epoch, int wait_ms, int* status,
                             unsigned int* cta_counter, cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || (D & 7) || (ldo & 7) || cap_recv <= 0) return ERR_BAD_SHAPE;
  EpPeers pt;
  fill_peers(pt, s);
  EpPlan plan{plan_ptrs[0], plan_ptrs[1], plan_ptrs[2], plan_ptrs[3], plan_ptrs[4], plan_ptrs[5], plan_ptrs[6]};
  ep_recv_kernel<<<cap_recv, 128, 0, st>>>(pt, off_recv, off_dflag, off_ddone, s->rank, s->world, E / s->world, D, plan,
                                           reinterpret_cast<__nv_bfloat16*>(out), ldo, epoch, spin_for(wait_ms), status,
                                           cta_counter);
  return static_cast<int>(cudaGetLastError());
}
