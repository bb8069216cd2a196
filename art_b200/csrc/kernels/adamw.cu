// Fused optimizer step over the flat fp32 LoRA buffers: global grad-norm clip + AdamW.
//
// All trainable parameters (every LoRA A and B) live in ONE contiguous fp32 master
// buffer with matching flat gradient / first-moment / second-moment buffers, so the
// optimizer is two launches regardless of how many adapters exist: a sum-of-squares
// reduction and the update.  The clip factor is computed on the device from the reduced
// norm (no host round trip), and the same flat gradient buffer is what the data-parallel
// all-reduce operates on.
//
// Replaces the reference's bitsandbytes paged 8-bit AdamW and HF grad clipping
// (src/art/dev/model.py:69-85: betas 0.9/0.99, weight decay 0.1, max_grad_norm 0.1;
// per-step learning rate forced at src/art/local/train.py:44-48).
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "host_utils.h"

namespace artb {

__global__ void sumsq_kernel(const float* __restrict__ g, long n, float scale, float* __restrict__ accum) {
  float s = 0.f;
  const long n4 = n >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    float4 v = g4[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const float v = g[(n4 << 2) + threadIdx.x];
    s += v * v;
  }
  s *= scale * scale;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  __shared__ float red[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = s;
  __syncthreads();
  if (warp == 0) {
    s = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) atomicAdd(accum, s);
  }
}

// stats[0] = sum of squares of (scaled) grads (input), stats[1] = grad norm (output, pre-clip)
__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, long n, float lr, float b1, float b2, float eps, float wd,
                             float bias1, float bias2, float max_norm, float grad_scale,
                             float* __restrict__ stats) {
  const float norm = sqrtf(stats[0]);
  if (blockIdx.x == 0 && threadIdx.x == 0) stats[1] = norm;
  float clip = 1.f;
  if (max_norm > 0.f) clip = fminf(1.f, max_norm / (norm + 1e-6f));
  const float gs = grad_scale * clip;
  const float step_size = lr / bias1;
  const float inv_sqrt_b2 = rsqrtf(bias2);
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const float gi = g[i] * gs;
    float pi = p[i] * (1.f - lr * wd);
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    pi -= step_size * mi / (sqrtf(vi) * inv_sqrt_b2 + eps);
    p[i] = pi;
  }
}

}  // namespace artb

using namespace artb;

// accum[0] += sum((scale * g)^2).  The caller zeroes accum before the first bucket.
ARTB_EXPORT int artb_grad_sumsq(const float* g, long n, float scale, float* accum, cudaStream_t st) {
  if (n <= 0) return 0;
  if (reinterpret_cast<uintptr_t>(g) & 15) return ERR_BAD_ALIGN;
  long blocks = (n / 4 + 255) / 256;
  long cap = static_cast<long>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  sumsq_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(g, n, scale, accum);
  return static_cast<int>(cudaGetLastError());
}

// One AdamW step (decoupled weight decay) on flat buffers.  `step` is 1-based.
// Gradients are multiplied by grad_scale and by the clip factor min(1, max_norm/(norm+1e-6)).
ARTB_EXPORT int artb_adamw_step(float* p, const float* g, float* m, float* v, long n, float lr, float b1, float b2,
                                float eps, float wd, int step, float max_norm, float grad_scale, float* stats,
                                cudaStream_t st) {
  if (n <= 0) return 0;
  const float bias1 = 1.f - powf(b1, static_cast<float>(step));
  const float bias2 = 1.f - powf(b2, static_cast<float>(step));
  long blocks = (n + 255) / 256;
  long cap = static_cast<long>(sm_count()) * 8;
  if (blocks > cap) blocks = cap;
  adamw_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(p, g, m, v, n, lr, b1, b2, eps, wd, bias1, bias2, max_norm,
                                                         grad_scale, stats);
  return static_cast<int>(cudaGetLastError());
}
