// Context parallelism for the tree-masked attention: K/V exchange and dK/dV reduction over NVLink.
//
// A packed row of S tokens is cut into 2P chunks; rank r owns chunks r and 2P-1-r (zig-zag, so the
// causal work is balanced).  All token-wise layers run on the local S/P tokens.  For attention every
// rank keeps a full-length [rows*S, ld] q|k|v buffer in symmetric memory:
//
//   kv_exchange   one CTA per local token: the whole q|k|v row goes to the token's global position
//                 in this rank's buffer, the k|v part also into every peer's buffer (16-byte stores
//                 over NVLink); the last CTA publishes an arrival flag to every peer
//   wait          bounded wait for the arrival flags of all peers (one tiny CTA)
//   -> the unchanged single-GPU attention kernels run on the full buffer with the tile-state rows
//      of non-local query blocks cleared, so each rank does exactly its own share of the tiles
//   dkv_push      backward: this rank's partial dK|dV for rows owned by a peer are pushed into the
//                 owner's staging slot [source]; last CTA publishes the flag
//   dkv_reduce    one CTA per local token: waits for the sources' flags, sums the partials in fp32
//                 (fixed order) with the local one, writes the local dq|dk|dv row
//
// Peers only ever store into a slot that its owner has finished with: the buffers are indexed by
// (layer, call parity) and a rank cannot run two calls ahead of a peer, because every call needs
// that peer's data (see parallel/cp.py).  Waits are bounded and report ST_TIMEOUT_PEER.
//
// The reference has no context parallelism: long sequences are one dense [B,S,S] bias on one GPU
// (src/art/local/train.py:177-215).  Unfused equivalent: NCCL all_gather of K/V + SDPA,
// reduce_scatter of dK/dV.
#include <cuda_bf16.h>

#include "host_utils.h"
#include "ptx_sm100.cuh"
#include "symm.cuh"

namespace artb {

constexpr int CP_MAX = 8;
struct CpPeers {
  char* base[CP_MAX];
};

__device__ __forceinline__ void cp_last_cta_flags(const CpPeers& pt, long off_flag, int rank, int P, uint32_t epoch,
                                                  unsigned int* cta_counter) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(cta_counter, 1u);
    if (prev + 1 == gridDim.x) {
      *cta_counter = 0;
      __threadfence_system();
      for (int p = 0; p < P; ++p) st_release_sys_u32(reinterpret_cast<uint32_t*>(pt.base[p] + off_flag) + rank, epoch);
    }
  }
}

__global__ void __launch_bounds__(128)
cp_kv_exchange_kernel(CpPeers pt, long off_full, long off_flag, int rank, int P, const uint4* __restrict__ local,
                      int ld16 /* row pitch of both buffers in 16-byte units */, int kv0_16, int row16,
                      const int* __restrict__ local_to_global, uint32_t epoch, unsigned int* cta_counter) {
  const int li = blockIdx.x;
  const long g = local_to_global[li];
  const uint4* src = local + static_cast<size_t>(li) * ld16;
  uint4* mine = reinterpret_cast<uint4*>(pt.base[rank] + off_full) + g * ld16;
  for (int i = threadIdx.x; i < row16; i += blockDim.x) {
    const uint4 v = src[i];
    mine[i] = v;
    if (i >= kv0_16) {
      for (int q = 1; q < P; ++q) {
        const int p = (rank + q) % P;
        (reinterpret_cast<uint4*>(pt.base[p] + off_full) + g * ld16)[i] = v;
      }
    }
  }
  cp_last_cta_flags(pt, off_flag, rank, P, epoch, cta_counter);
}

__global__ void cp_wait_kernel(CpPeers pt, long off_flag, int rank, int P, uint32_t epoch, uint32_t spin, int* status) {
  if (threadIdx.x < P && threadIdx.x != rank) {
    if (!wait_flag_ge(reinterpret_cast<const uint32_t*>(pt.base[rank] + off_flag) + threadIdx.x, epoch, spin))
      atomicMax(status, ST_TIMEOUT_PEER);
  }
}

// full: dq|dk|dv [rows*S, ld]; rows owned by a peer send their dk|dv part to stage[me][local index at owner].
__global__ void __launch_bounds__(128)
cp_dkv_push_kernel(CpPeers pt, long off_stage, long off_flag, int rank, int P, const uint4* __restrict__ full, int ld16,
                   int kv0_16, int kv16, const int* __restrict__ owner_of, const int* __restrict__ local_index_of,
                   long n_local, uint32_t epoch, unsigned int* cta_counter) {
  const long g = blockIdx.x;
  const int o = owner_of[g];
  if (o != rank) {
    const uint4* src = full + g * ld16 + kv0_16;
    uint4* dst = reinterpret_cast<uint4*>(pt.base[o] + off_stage) +
                 (static_cast<size_t>(rank) * n_local + local_index_of[g]) * kv16;
    for (int i = threadIdx.x; i < kv16; i += blockDim.x) dst[i] = src[i];
  }
  cp_last_cta_flags(pt, off_flag, rank, P, epoch, cta_counter);
}

__global__ void __launch_bounds__(128)
cp_dkv_reduce_kernel(CpPeers pt, long off_stage, long off_flag, int rank, int P, const uint4* __restrict__ full,
                     int ld16, int kv0_16, int kv16, const int* __restrict__ local_to_global, long n_local,
                     uint4* __restrict__ out, int ldo16, uint32_t epoch, uint32_t spin, int* status) {
  const int li = blockIdx.x;
  const long g = local_to_global[li];
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int p = 0; p < P; ++p)
      if (p != rank && !wait_flag_ge(reinterpret_cast<const uint32_t*>(pt.base[rank] + off_flag) + p, epoch, spin))
        ok = 0;
    if (!ok) atomicMax(status, ST_TIMEOUT_PEER);
    s_ok = ok;
  }
  __syncthreads();
  const uint4* src = full + g * ld16;
  uint4* dst = out + static_cast<size_t>(li) * ldo16;
  for (int i = threadIdx.x; i < kv0_16; i += blockDim.x) dst[i] = src[i];   // dq: local only
  if (!s_ok) return;
  const uint4* stage = reinterpret_cast<const uint4*>(pt.base[rank] + off_stage);
  for (int i = threadIdx.x; i < kv16; i += blockDim.x) {
    float acc[8];
    {
      const uint4 v = src[kv0_16 + i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    for (int p = 0; p < P; ++p) {
      if (p == rank) continue;
      const uint4 v = __ldcg(stage + (static_cast<size_t>(p) * n_local + li) * kv16 + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 ov;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    dst[kv0_16 + i] = ov;
  }
}

static void cp_fill(CpPeers& pt, const SymmState* s) {
  for (int p = 0; p < CP_MAX; ++p) pt.base[p] = p < s->world ? static_cast<char*>(s->table.base[p]) : nullptr;
}
static uint32_t cp_spin(int wait_ms) {
  return static_cast<uint32_t>(wait_ms <= 0 ? 2000000 : static_cast<long>(wait_ms) * 1000);
}

}  // namespace artb

using namespace artb;

// local bf16 [n_local, ld] -> symmetric full buffer [n_global, ld] at off_full (own rows: q|k|v; peers: k|v).
// kv0 = first k column (elements), ld / kv0 multiples of 8.  Then waits for every peer's arrival flag.
ARTB_EXPORT int artb_cp_kv_exchange(void* h, long off_full, long off_flag, const void* local, int ld, int kv0,
                                    const int* local_to_global, int n_local, unsigned int epoch, int wait_ms,
                                    unsigned int* cta_counter, int* status, cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || s->world > CP_MAX || (ld & 7) || (kv0 & 7) || n_local <= 0) return ERR_BAD_SHAPE;
  CpPeers pt;
  cp_fill(pt, s);
  cp_kv_exchange_kernel<<<n_local, 128, 0, st>>>(pt, off_full, off_flag, s->rank, s->world,
                                                reinterpret_cast<const uint4*>(local), ld / 8, kv0 / 8, ld / 8,
                                                local_to_global, epoch, cta_counter);
  cp_wait_kernel<<<1, 32, 0, st>>>(pt, off_flag, s->rank, s->world, epoch, cp_spin(wait_ms), status);
  return static_cast<int>(cudaGetLastError());
}

// full bf16 [n_global, ld] private (dq|dk|dv partials) -> out bf16 [n_local, ldo] with dk|dv summed over ranks.
ARTB_EXPORT int artb_cp_dkv_reduce(void* h, long off_stage, long off_flag, const void* full, int ld, int kv0,
                                   const int* owner_of, const int* local_index_of, const int* local_to_global,
                                   long n_global, int n_local, void* out, int ldo, unsigned int epoch, int wait_ms,
                                   unsigned int* cta_counter, int* status, cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || s->world > CP_MAX || (ld & 7) || (kv0 & 7) || (ldo & 7) || n_local <= 0) return ERR_BAD_SHAPE;
  CpPeers pt;
  cp_fill(pt, s);
  const int kv16 = (ld - kv0) / 8;
  cp_dkv_push_kernel<<<static_cast<unsigned>(n_global), 128, 0, st>>>(pt, off_stage, off_flag, s->rank, s->world,
                                                                      reinterpret_cast<const uint4*>(full), ld / 8,
                                                                      kv0 / 8, kv16, owner_of, local_index_of, n_local,
                                                                      epoch, cta_counter);
  cp_dkv_reduce_kernel<<<n_local, 128, 0, st>>>(pt, off_stage, off_flag, s->rank, s->world,
                                                reinterpret_cast<const uint4*>(full), ld / 8, kv0 / 8, kv16,
                                                local_to_global, n_local, reinterpret_cast<uint4*>(out), ldo / 8, epoch,
                                                cp_spin(wait_ms), status);
  return static_cast<int>(cudaGetLastError());
}
