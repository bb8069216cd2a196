// Decode-side tensor parallelism: finalize of the split-K weight-streaming GEMM fused with a one-shot
// all-reduce over NVLink, and the LoRA hand-off push.
//
//   splitk_finalize_allreduce   every rank holds an fp32 partial [M, N] (its slice of the reduction dimension,
//       accumulated by the split-K GEMM).  One persistent kernel per rank: every CTA stores its 4 KB slices into the
//       peers' staging slot [rank], publishes one flag per peer, waits (bounded) for the flag of the same-index CTA
//       of every peer, then adds the staged slices + bias + residual, writes bf16 and re-zeroes the workspace.  For decode shapes
//       (M <= 256 rows, 2.6 MB per all-reduce, 128 of them per step) the exchange is latency-bound, so it rides on
//       a kernel that has to run anyway instead of a separate collective launch.
//   lora_push / lora_wait       the trainer rank stores its flat LoRA buffer into the engine ranks' symmetric
//       buffers (device-memory hand-off, no disk round trip) and publishes an epoch; receivers wait bounded.
//
// Staging is indexed by call parity; a peer can only be two calls ahead after this rank's flags of the call in
// between were published, i.e. after this rank finished reading the slot.  Plain ld/st only, no multimem.
//
// Reference: the inference library's custom all-reduce is reached only through `tensor_parallel_size`
// (src/art/dev/engine.py:27); adapters are handed over through safetensors files on disk
// (src/art/local/service.py:150-174).
#include <cuda_bf16.h>

#include "host_utils.h"
#include "ptx_sm100.cuh"
#include "symm.cuh"

namespace artb {

constexpr int AR_MAX = 8;
constexpr int AR_SLICE = 1024;   // floats per slice: 256 threads x float4

struct ArPeers {
  char* base[AR_MAX];
};

__global__ void __launch_bounds__(256)
splitk_finalize_allreduce_kernel(ArPeers pt, long off_stage, long off_flag, int rank, int P, float* __restrict__ ws,
                                 long n /* floats, multiple of 4 */, int N, const float* __restrict__ bias,
                                 const __nv_bfloat16* __restrict__ R, int ldr, int res_cols,
                                 __nv_bfloat16* __restrict__ out, int ldc, long stage_stride, int n_slices,
                                 uint32_t epoch, uint32_t spin, int* status) {
  __shared__ int s_ok;
  // phase 1: push every slice this CTA owns to all peers, then ONE flag per (CTA, peer): the CTA with the same index on
  // the peer owns the same slices (same grid on every rank), so a single NVLink round trip covers the whole kernel
  for (int sl = blockIdx.x; sl < n_slices; sl += gridDim.x) {
    const long i = static_cast<long>(sl) * AR_SLICE + threadIdx.x * 4;
    if (i < n) {
      const float4 v = *reinterpret_cast<const float4*>(ws + i);
      for (int q = 1; q < P; ++q) {
        const int p = (rank + q) % P;
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(pt.base[p] + off_stage) + rank * stage_stride + i) = v;
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int q = 1; q < P; ++q) {
      const int p = (rank + q) % P;
      st_release_sys_u32(reinterpret_cast<uint32_t*>(pt.base[p] + off_flag) + static_cast<size_t>(rank) * gridDim.x + blockIdx.x,
                         epoch);
    }
    for (int q = 1; q < P; ++q) {
      const int p = (rank + q) % P;
      if (!wait_flag_ge(reinterpret_cast<const uint32_t*>(pt.base[rank] + off_flag) + static_cast<size_t>(p) * gridDim.x + blockIdx.x,
                        epoch, spin))
        ok = 0;
    }
    if (!ok) atomicMax(status, ST_TIMEOUT_PEER);
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  // phase 2: local partial + the peers' staged partials (+ bias, residual) -> bf16; the workspace is re-zeroed
  for (int sl = blockIdx.x; sl < n_slices; sl += gridDim.x) {
    const long i = static_cast<long>(sl) * AR_SLICE + threadIdx.x * 4;
    if (i >= n) continue;
    float4 v = *reinterpret_cast<float4*>(ws + i);
    *reinterpret_cast<float4*>(ws + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < P; ++p) {
      if (p == rank) continue;
      const float4 o = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(pt.base[rank] + off_stage) +
                                                              p * stage_stride + i));
      v.x += o.x;
      v.y += o.y;
      v.z += o.z;
      v.w += o.w;
    }
    const long m = i / N;
    const int c = static_cast<int>(i - m * N);
    if (bias) {
      v.x += bias[c];
      v.y += bias[c + 1];
      v.z += bias[c + 2];
      v.w += bias[c + 3];
    }
    if (R && c < res_cols) {
      const __nv_bfloat16* r = R + m * ldr + c;
      v.x += __bfloat162float(r[0]);
      v.y += __bfloat162float(r[1]);
      v.z += __bfloat162float(r[2]);
      v.w += __bfloat162float(r[3]);
    }
    uint2 o2;
    o2.x = pack_bf16x2(v.x, v.y);
    o2.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(out + m * ldc + c) = o2;
  }
}

__global__ void __launch_bounds__(256)
lora_push_kernel(ArPeers pt, long off_data, long off_flag, int rank, int P, const float4* __restrict__ src, long n4,
                 uint32_t epoch, unsigned int* cta_counter) {
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float4 v = src[i];
    for (int q = 1; q < P; ++q) reinterpret_cast<float4*>(pt.base[(rank + q) % P] + off_data)[i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(cta_counter, 1u);
    if (prev + 1 == gridDim.x) {
      *cta_counter = 0;
      __threadfence_system();
      for (int q = 1; q < P; ++q)
        st_release_sys_u32(reinterpret_cast<uint32_t*>(pt.base[(rank + q) % P] + off_flag) + rank, epoch);
    }
  }
}

__global__ void lora_wait_kernel(ArPeers pt, long off_flag, int rank, int src, uint32_t epoch, uint32_t spin, int* status) {
  if (threadIdx.x == 0 &&
      !wait_flag_ge(reinterpret_cast<const uint32_t*>(pt.base[rank] + off_flag) + src, epoch, spin))
    atomicMax(status, ST_TIMEOUT_PEER);
}

static void ar_fill(ArPeers& pt, const SymmState* s) {
  for (int p = 0; p < AR_MAX; ++p) pt.base[p] = p < s->world ? static_cast<char*>(s->table.base[p]) : nullptr;
}
static uint32_t ar_spin(int wait_ms) {
  return static_cast<uint32_t>(wait_ms <= 0 ? 2000000 : static_cast<long>(wait_ms) * 1000);
}

}  // namespace artb

using namespace artb;

// ws fp32 [M, N] dense (ldw == N, M*N % 4 == 0): this rank's partial; out = bf16(sum over ranks + bias + residual).
// Symmetric layout: staging fp32 [P][stage_stride] at off_stage (stage_stride >= M*N), flags uint32 [P][grid <= SM count].
ARTB_EXPORT int artb_splitk_finalize_allreduce(void* h, long off_stage, long off_flag, long stage_stride, float* ws, int M,
                                               int N, const float* bias, const void* R, int ldr, int res_cols, void* out,
                                               int ldc, unsigned int epoch, int wait_ms, int* status, cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  const long n = static_cast<long>(M) * N;
  if (!s || s->world > AR_MAX || M <= 0 || (N & 3) || n > stage_stride) return ERR_BAD_SHAPE;
  ArPeers pt;
  ar_fill(pt, s);
  const int n_slices = static_cast<int>((n + AR_SLICE - 1) / AR_SLICE);
  int grid = n_slices < sm_count() ? n_slices : sm_count();   // persistent: every CTA's partner on a peer is resident too
  splitk_finalize_allreduce_kernel<<<grid, 256, 0, st>>>(pt, off_stage, off_flag, s->rank, s->world, ws, n, N, bias,
                                                         reinterpret_cast<const __nv_bfloat16*>(R), ldr,
                                                         res_cols > 0 ? res_cols : N, reinterpret_cast<__nv_bfloat16*>(out),
                                                         ldc, stage_stride, n_slices, epoch, ar_spin(wait_ms), status);
  return static_cast<int>(cudaGetLastError());
}

// Broadcast n floats (multiple of 4) from this rank's private buffer into every peer's symmetric buffer at off_data.
ARTB_EXPORT int artb_lora_push(void* h, long off_data, long off_flag, const float* src, long n, unsigned int epoch,
                               unsigned int* cta_counter, cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || s->world > AR_MAX || n <= 0 || (n & 3)) return ERR_BAD_SHAPE;
  ArPeers pt;
  ar_fill(pt, s);
  const long n4 = n >> 2;
  int grid = static_cast<int>((n4 + 255) / 256);
  if (grid > 2 * sm_count()) grid = 2 * sm_count();
  lora_push_kernel<<<grid, 256, 0, st>>>(pt, off_data, off_flag, s->rank, s->world, reinterpret_cast<const float4*>(src), n4,
                                        epoch, cta_counter);
  return static_cast<int>(cudaGetLastError());
}

ARTB_EXPORT int artb_lora_wait(void* h, long off_flag, int src, unsigned int epoch, int wait_ms, int* status,
                               cudaStream_t st) {
  auto* s = static_cast<SymmState*>(h);
  if (!s || src < 0 || src >= s->world) return ERR_BAD_SHAPE;
  ArPeers pt;
  ar_fill(pt, s);
  lora_wait_kernel<<<1, 32, 0, st>>>(pt, off_flag, s->rank, src, epoch, ar_spin(wait_ms), status);
  return static_cast<int>(cudaGetLastError());
}
