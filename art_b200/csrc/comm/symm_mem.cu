// Symmetric memory over CUDA IPC + the NVLink collectives built on it.
//
// Every rank allocates the same-sized device buffer (data area followed by a signal pad of
// 64-bit epoch counters), exports it with cudaIpcGetMemHandle, and maps every peer's buffer;
// kernels then receive a table of peer base pointers and read / write remote memory with plain
// ld/st over NVLink (no TMA, no multicast).  Synchronisation between GPUs uses monotonically
// increasing epochs in the signal pads: a rank publishes epoch e to slot [its rank] of every
// peer's pad (st.release.sys after a system fence) and waits (ld.acquire.sys) until all slots of
// its own pad reach e.  Every wait is bounded; on expiry the kernel records ST_TIMEOUT_PEER in
// the status word and returns, so a missing peer surfaces as a host-side error, not a hang.
//
// lora_grad_allreduce: two-shot all-reduce of the flat fp32 LoRA-gradient buffer.  Rank r sums
// slice r over all peers' buffers (remote loads), scales it, and stores the result into slice r
// of every peer (remote stores); epoch barriers precede the loads and follow the stores.  One
// cooperative kernel per rank does all of it.
//
// The reference has no collective of any kind (single GPU); this file serves the multi-GPU
// configurations (data-parallel LoRA gradient sync).
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "host_utils.h"
#include "ptx_sm100.cuh"
#include "symm.cuh"

namespace cg = cooperative_groups;

namespace artb {

// Executed by the first `world` threads of ONE block.  Returns false on timeout.
__device__ __forceinline__ bool epoch_barrier(const PeerTable& pt, int rank, int world, int channel, uint64_t epoch,
                                              uint32_t spin_limit) {
  const int q = threadIdx.x;
  bool ok = true;
  if (q < world) {
    __threadfence_system();
    st_release_sys(pt.pad[q] + channel * MAX_RANKS + rank, epoch);
    const uint64_t* mine = pt.pad[rank] + channel * MAX_RANKS + q;
    WaitBudget w(spin_limit);      // microseconds
    while (ld_acquire_sys(mine) < epoch) {
      if (w.expired()) {
        ok = false;
        break;
      }
      __nanosleep(64);
    }
  }
  return ok;
}

// grid-wide: block 0 runs the cross-GPU barrier, a cooperative grid sync releases the other
// blocks.  `fail` is a device-local sticky flag set when a wait expired.
__device__ bool grid_epoch_barrier(const PeerTable& pt, int rank, int world, int channel, uint64_t epoch,
                                   uint32_t spin_limit, volatile uint32_t* fail, int* status) {
  __shared__ int s_ok;
  cg::grid_group grid = cg::this_grid();
  grid.sync();                       // every block's earlier stores are issued before the epoch is published
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (!epoch_barrier(pt, rank, world, channel, epoch, spin_limit)) s_ok = 0;
    __syncthreads();
    if (threadIdx.x == 0 && !s_ok) {
      atomicMax(status, ST_TIMEOUT_PEER);
      *fail = 1;
      __threadfence();
    }
  }
  grid.sync();
  __threadfence_system();
  return *fail == 0;
}

__global__ void __launch_bounds__(512)
lora_grad_allreduce_kernel(PeerTable pt, int rank, int world, long n, float scale, uint64_t epoch, uint32_t spin_limit,
                           uint32_t* gate, int* status) {
  // phase 0: everyone's gradients are in place
  if (!grid_epoch_barrier(pt, rank, world, 0, 2 * epoch, spin_limit, gate, status)) return;
  // phase 1+2: reduce my slice over all ranks, scale, broadcast it
  const long n4 = n >> 2;                       // float4 units (n is padded to a multiple of 4 * world)
  const long per = n4 / world;
  const long lo = per * rank, hi = (rank == world - 1) ? n4 : lo + per;
  for (long i = lo + blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < hi;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int q = 0; q < world; ++q) {
      const int src = (rank + q) % world;       // stagger peers so links are used evenly
      const float4 v = reinterpret_cast<const float4*>(pt.base[src])[i];
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    acc.x *= scale;
    acc.y *= scale;
    acc.z *= scale;
    acc.w *= scale;
#pragma unroll 4
    for (int q = 0; q < world; ++q) {
      const int dst = (rank + q) % world;
      reinterpret_cast<float4*>(pt.base[dst])[i] = acc;
    }
  }
  // phase 3: all slices have landed everywhere
  __threadfence_system();
  grid_epoch_barrier(pt, rank, world, 0, 2 * epoch + 1, spin_limit, gate, status);
}


}  // namespace artb

using namespace artb;

// ---- host API -------------------------------------------------------------------------------------------------
// 1. h = artb_symm_create(rank, world, data_bytes)         allocates data + pad on the current device
// 2. artb_symm_export(h, handle64)                          64-byte IPC handle to send to the peers
// 3. artb_symm_import(h, peer_rank, handle64)               map a peer (call for every peer)
// 4. artb_symm_local_ptr(h) / kernels
// 5. artb_symm_destroy(h)
ARTB_EXPORT void* artb_symm_create(int rank, int world, size_t data_bytes) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return nullptr;
  auto* s = new SymmState();
  s->rank = rank;
  s->world = world;
  s->data_bytes = (data_bytes + 255) & ~static_cast<size_t>(255);
  const size_t total = s->data_bytes + PAD_SLOTS * sizeof(uint64_t);
  if (cudaMalloc(&s->local, total) != cudaSuccess) {
    delete s;
    return nullptr;
  }
  cudaMemset(s->local, 0, total);
  cudaMalloc(&s->gate, 2 * sizeof(uint32_t));   // [0]: sticky failure flag of this rank's kernels
  cudaMemset(s->gate, 0, 2 * sizeof(uint32_t));
  memset(&s->table, 0, sizeof(s->table));
  memset(s->opened, 0, sizeof(s->opened));
  s->table.base[rank] = s->local;
  s->table.pad[rank] = reinterpret_cast<uint64_t*>(static_cast<char*>(s->local) + s->data_bytes);
  cudaDeviceSynchronize();
  return s;
}

ARTB_EXPORT int artb_symm_export(void* h, void* handle64) {
  auto* s = static_cast<SymmState*>(h);
  cudaIpcMemHandle_t hd;
  cudaError_t e = cudaIpcGetMemHandle(&hd, s->local);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle64, &hd, sizeof(hd));
  return 0;
}

ARTB_EXPORT int artb_symm_import(void* h, int peer, const void* handle64) {
  auto* s = static_cast<SymmState*>(h);
  if (peer < 0 || peer >= s->world) return ERR_BAD_SHAPE;
  if (peer == s->rank) return 0;
  cudaIpcMemHandle_t hd;
  memcpy(&hd, handle64, sizeof(hd));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return static_cast<int>(e);
  s->opened[peer] = p;
  s->table.base[peer] = p;
  s->table.pad[peer] = reinterpret_cast<uint64_t*>(static_cast<char*>(p) + s->data_bytes);
  return 0;
}

ARTB_EXPORT void* artb_symm_local_ptr(void* h) { return static_cast<SymmState*>(h)->local; }
ARTB_EXPORT void* artb_symm_peer_ptr(void* h, int peer) { return static_cast<SymmState*>(h)->table.base[peer]; }

ARTB_EXPORT void artb_symm_destroy(void* h) {
  auto* s = static_cast<SymmState*>(h);
  if (!s) return;
  cudaDeviceSynchronize();
  for (int q = 0; q < s->world; ++q)
    if (s->opened[q]) cudaIpcCloseMemHandle(s->opened[q]);
  cudaFree(s->gate);
  cudaFree(s->local);
  delete s;
}

// In-place all-reduce (sum, then * scale) of the first n floats of the symmetric data area.
// n must be a multiple of 4 * world.  wait_ms bounds every device-side wait.
ARTB_EXPORT int artb_lora_grad_allreduce(void* h, long n, float scale, int wait_ms, int* status, cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  if (n <= 0 || n % (4L * s->world) || static_cast<size_t>(n) * 4 > s->data_bytes) return ERR_BAD_SHAPE;
  s->epoch += 1;
  int rank = s->rank, world = s->world;
  uint64_t epoch = s->epoch;
  // each poll sleeps ~64 ns (plus the load round trip, >= 1 us over NVLink): ~1 us per poll
  uint32_t spin = static_cast<uint32_t>(wait_ms <= 0 ? 2000000 : static_cast<long>(wait_ms) * 1000);
  int threads = 512;
  long slice4 = (n / 4) / world;
  int blocks = static_cast<int>((slice4 + threads - 1) / threads);
  int cap = sm_count();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  PeerTable pt = s->table;
  uint32_t* gate = s->gate;
  void* args[] = {&pt, &rank, &world, &n, &scale, &epoch, &spin, &gate, &status};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(lora_grad_allreduce_kernel), dim3(blocks),
                                              dim3(threads), args, 0, st);
  return static_cast<int>(e);
}

// Clear the sticky failure flag after the host has handled a reported timeout.
ARTB_EXPORT void artb_symm_reset(void* h) {
  auto* s = static_cast<SymmState*>(h);
  cudaMemset(s->gate, 0, 2 * sizeof(uint32_t));
}
