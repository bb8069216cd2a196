// Top-k / top-p (nucleus) sampling over materialised logits, one CTA per row.
//
// The fused LM-head sampler (logprob_loss.cu: EpiSample) never writes logits, which is what the common
// temperature-only request wants.  A request that restricts the support needs a per-row threshold first, so this
// path takes fp32 logits [M, V] (one plain GEMM) and does, per row, with x = logit / temperature:
//
//   1. max and sum of exp            -> log Z of the full distribution
//      min-p:  keep x >= max + log(min_p), i.e. tokens at least min_p times as likely as the best one
//   2. top-k:  the k-th largest x by a 4-pass radix select (8 bits per pass) over an order-preserving integer key;
//              per-warp shared-memory histograms keep the atomics local
//   3. top-p:  among the survivors of 2, the largest threshold whose tail mass still reaches p x (surviving mass):
//              the same radix walk over histograms of exp(x - max) instead of counts
//   4. Gumbel-max over the survivors with the same counter-based noise as the fused sampler
//
// Order of the two filters and the renormalisation between them follow the usual serving convention (top-k first,
// top-p on what is left).  Values equal to a threshold are all kept.  The reported log-probability is that of the
// token under the temperature-scaled FULL distribution, as in the fused sampler, so that a trainer that recomputes
// log-probabilities sees the same quantity whatever the sampling restriction was.
//
// Reference: the reference delegates sampling to vLLM (src/art/vllm/server.py); there is no kernel of its own.
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "host_utils.h"
#include "sampling.cuh"

namespace artb {

constexpr int SR_THREADS = 512;
constexpr int SR_WARPS = SR_THREADS / 32;

struct SrShared {
  float hist[SR_WARPS][256];
  float red[SR_WARPS];
  int red_i[SR_WARPS];
  float red_x[SR_WARPS];
  float bcast_f;
  uint32_t bcast_u;
};

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return b ^ ((b >> 31) ? 0xffffffffu : 0x80000000u);   // larger float <=> larger unsigned key
}

// f(index, raw logit) over one row, block-strided; 16-byte loads when the row allows it (each thread still visits its
// indices in ascending order).
template <class F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ x, int V, bool vec, F f) {
  const int tid = threadIdx.x;
  if (vec) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int n4 = V >> 2;
    for (int i = tid; i < n4; i += SR_THREADS) {
      const float4 q = x4[i];
      f(4 * i, q.x);
      f(4 * i + 1, q.y);
      f(4 * i + 2, q.z);
      f(4 * i + 3, q.w);
    }
    for (int v = (n4 << 2) + tid; v < V; v += SR_THREADS) f(v, x[v]);
  } else {
    for (int v = tid; v < V; v += SR_THREADS) f(v, x[v]);
  }
}

__device__ float block_max(float v, SrShared& s) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s.red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = s.red[0];
    for (int w = 1; w < SR_WARPS; ++w) m = fmaxf(m, s.red[w]);
    s.bcast_f = m;
  }
  __syncthreads();
  return s.bcast_f;
}

__device__ float block_sum(float v, SrShared& s) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) s.red[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int w = 0; w < SR_WARPS; ++w) m += s.red[w];
    s.bcast_f = m;
  }
  __syncthreads();
  return s.bcast_f;
}

// Largest key t such that the total weight of {v : key_v >= max(t, floor_key)} reaches `target`; weight = 1 (MASS =
// false: t is the target-th largest key) or exp(x - mx).  Four passes of 8 bits from the top.
template <bool MASS>
__device__ uint32_t radix_select(const float* __restrict__ x, int V, bool vec, float sc, float mx, uint32_t floor_key,
                                 float target, SrShared& s) {
  const int tid = threadIdx.x, warp = tid >> 5;
  uint32_t prefix = 0;
  float remaining = target;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < SR_WARPS * 256; i += SR_THREADS) (&s.hist[0][0])[i] = 0.f;
    __syncthreads();
    const uint32_t himask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
    for_each_logit(x, V, vec, [&](int, float raw) {
      const float xs = raw * sc;
      const uint32_t key = order_key(xs);
      if (key >= floor_key && (key & himask) == prefix)
        atomicAdd(&s.hist[warp][(key >> shift) & 255u], MASS ? __expf(xs - mx) : 1.f);
    });
    __syncthreads();
    if (tid < 256) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < SR_WARPS; ++w) t += s.hist[w][tid];
      s.hist[0][tid] = t;
    }
    __syncthreads();
    if (tid == 0) {
      float cum = 0.f;
      int sel = -1, lowest = 0;
      for (int b = 255; b >= 0; --b) {
        const float h = s.hist[0][b];
        if (h > 0.f) lowest = b;
        if (sel < 0 && cum + h >= remaining && h > 0.f) {
          sel = b;
          s.bcast_f = remaining - cum;
        }
        if (sel < 0) cum += h;
      }
      if (sel < 0) {   // rounding left the target just out of reach: keep everything that matches the prefix
        sel = lowest;
        s.bcast_f = 0.f;
      }
      s.bcast_u = prefix | (static_cast<uint32_t>(sel) << shift);
    }
    __syncthreads();
    prefix = s.bcast_u;
    remaining = s.bcast_f;
    __syncthreads();
  }
  return prefix;
}

__global__ void __launch_bounds__(SR_THREADS)
sample_restricted_kernel(const float* __restrict__ logits, long ld, const float* __restrict__ inv_temp,
                         const uint32_t* __restrict__ row_seed, const int* __restrict__ top_k,
                         const float* __restrict__ top_p, const float* __restrict__ min_p, int M, int V,
                         int vocab_offset, int* __restrict__ token, float* __restrict__ logprob) {
  __shared__ SrShared s;
  const int row = blockIdx.x, tid = threadIdx.x;
  if (row >= M) return;
  const float* x = logits + static_cast<size_t>(row) * ld;
  const float it = inv_temp[row];
  const bool greedy = it == 0.f;
  const float sc = greedy ? 1.f : it;
  const bool vec = ((ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  float lm = -INFINITY;
  for_each_logit(x, V, vec, [&](int, float raw) { lm = fmaxf(lm, raw * sc); });
  const float mx = block_max(lm, s);
  float ls = 0.f;
  for_each_logit(x, V, vec, [&](int, float raw) { ls += __expf(raw * sc - mx); });
  const float Z = block_sum(ls, s);

  uint32_t tau = 0u;
  if (!greedy) {
    const int k = top_k[row];
    const float p = top_p[row];
    const float mp = min_p ? min_p[row] : 0.f;
    if (mp > 0.f) tau = order_key(mx + __logf(fminf(mp, 1.f)));
    if (k > 0 && k < V) {
      const uint32_t tk = radix_select<false>(x, V, vec, sc, mx, 0u, static_cast<float>(k), s);
      tau = tk > tau ? tk : tau;
    }
    if (p < 1.f) {
      float Zk = Z;
      if (tau) {
        float part = 0.f;
        for_each_logit(x, V, vec, [&](int, float raw) {
          const float xs = raw * sc;
          if (order_key(xs) >= tau) part += __expf(xs - mx);
        });
        Zk = block_sum(part, s);
      }
      const uint32_t tp = radix_select<true>(x, V, vec, sc, mx, tau, fmaxf(p, 0.f) * Zk, s);
      tau = tp > tau ? tp : tau;
    }
  }

  const uint32_t seed = row_seed[row];
  float best = -INFINITY, best_x = 0.f;
  int best_i = -1;
  for_each_logit(x, V, vec, [&](int v, float raw) {
    const float xs = raw * sc;
    if (order_key(xs) < tau) return;
    float score = xs;
    if (!greedy) score += gumbel_noise(seed, static_cast<uint32_t>(row), static_cast<uint32_t>(vocab_offset + v));
    if (score > best) {
      best = score;
      best_x = xs;
      best_i = v;
    }
  });
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const float ox = __shfl_xor_sync(0xffffffffu, best_x, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi >= 0 && (best_i < 0 || oi < best_i))) {
      best = ob;
      best_x = ox;
      best_i = oi;
    }
  }
  __syncthreads();
  if ((tid & 31) == 0) {
    s.red[tid >> 5] = best;
    s.red_x[tid >> 5] = best_x;
    s.red_i[tid >> 5] = best_i;
  }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < SR_WARPS; ++w)
      if (s.red[w] > best || (s.red[w] == best && s.red_i[w] >= 0 && (best_i < 0 || s.red_i[w] < best_i))) {
        best = s.red[w];
        best_x = s.red_x[w];
        best_i = s.red_i[w];
      }
    token[row] = vocab_offset + best_i;
    logprob[row] = best_x - (mx + logf(Z));
  }
}

// Sparse in-place logit edits before sampling: entry e rewrites logits[row[e], tok[e]] as
//   x = x > 0 ? x * mul_pos[e] : x * mul_neg[e];  x -= sub[e]
// which covers the repetition penalty (mul_pos = 1/p, mul_neg = p on every token of prompt + output), the frequency /
// presence penalties (sub = f * count + p on output tokens) and logit_bias (sub = -bias).  The host merges all edits of
// one (row, token) pair into one entry, so entries never collide.
__global__ void logit_adjust_kernel(float* logits, long ld, const int* row, const int* tok, const float* mul_pos,
                                    const float* mul_neg, const float* sub, int n, int M, int V) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const int r = row[e], t = tok[e];
  if (r < 0 || r >= M || t < 0 || t >= V) return;
  float* p = logits + static_cast<long>(r) * ld + t;
  float x = *p;
  x = x > 0.f ? x * mul_pos[e] : x * mul_neg[e];
  *p = x - sub[e];
}

// The k most likely tokens of every row with their log-probabilities under softmax(logits * inv_temp) (inv_temp 0:
// temperature 1 for reporting, as the greedy log-prob is reported): k rounds of a block-wide arg-max over values below
// the previous pick (ties broken by the smaller index).  k is small (<= 20); one CTA per row.
__global__ void __launch_bounds__(256) top_logprobs_kernel(const float* logits, long ld, const float* inv_temp, int M, int V,
                                                           int k, int* out_tok, float* out_lp) {
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* x = logits + static_cast<long>(r) * ld;
  float it = inv_temp ? inv_temp[r] : 1.f;
  if (it <= 0.f) it = 1.f;
  __shared__ float s_v[256];
  __shared__ int s_i[256];
  __shared__ float s_mx, s_lse;
  // log-sum-exp of the row
  float mx = -INFINITY;
  for (int j = tid; j < V; j += 256) mx = fmaxf(mx, x[j] * it);
  s_v[tid] = mx;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) s_v[tid] = fmaxf(s_v[tid], s_v[tid + o]);
    __syncthreads();
  }
  if (tid == 0) s_mx = s_v[0];
  __syncthreads();
  mx = s_mx;
  float z = 0.f;
  for (int j = tid; j < V; j += 256) z += __expf(x[j] * it - mx);
  s_v[tid] = z;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) s_v[tid] += s_v[tid + o];
    __syncthreads();
  }
  if (tid == 0) s_lse = mx + logf(s_v[0]);
  __syncthreads();
  float prev_v = INFINITY;
  int prev_i = -1;
  for (int round = 0; round < k; ++round) {
    float bv = -INFINITY;
    int bi = V;
    for (int j = tid; j < V; j += 256) {
      const float v = x[j] * it;
      const bool below = v < prev_v || (v == prev_v && j > prev_i);
      if (below && (v > bv || (v == bv && j < bi))) {
        bv = v;
        bi = j;
      }
    }
    s_v[tid] = bv;
    s_i[tid] = bi;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
      if (tid < o) {
        const float ov = s_v[tid + o];
        const int oi = s_i[tid + o];
        if (ov > s_v[tid] || (ov == s_v[tid] && oi < s_i[tid])) {
          s_v[tid] = ov;
          s_i[tid] = oi;
        }
      }
      __syncthreads();
    }
    prev_v = s_v[0];
    prev_i = s_i[0];
    if (tid == 0) {
      out_tok[r * k + round] = prev_i < V ? prev_i : -1;
      out_lp[r * k + round] = prev_i < V ? prev_v - s_lse : -INFINITY;
    }
    __syncthreads();
  }
}

}  // namespace artb

using namespace artb;

// logits fp32 [M, V] (row stride ld elements); top_k <= 0, top_p >= 1 and min_p <= 0 (or a null min_p) leave a row
// unrestricted.
ARTB_EXPORT int artb_sample_restricted(const float* logits, long ld, const float* inv_temp, const uint32_t* row_seed,
                                       const int* top_k, const float* top_p, const float* min_p, int M, int V,
                                       int vocab_offset, int* token, float* logprob, cudaStream_t stream) {
  if (M <= 0) return 0;
  if (V <= 0 || ld < V) return ERR_BAD_SHAPE;
  sample_restricted_kernel<<<M, SR_THREADS, 0, stream>>>(logits, ld, inv_temp, row_seed, top_k, top_p, min_p, M, V,
                                                         vocab_offset, token, logprob);
  return static_cast<int>(cudaGetLastError());
}

// In-place sparse logit edits (penalties, logit_bias); see logit_adjust_kernel.
ARTB_EXPORT int artb_logit_adjust(float* logits, long ld, const int* row, const int* tok, const float* mul_pos,
                                  const float* mul_neg, const float* sub, int n, int M, int V, cudaStream_t stream) {
  if (n <= 0 || M <= 0) return 0;
  if (V <= 0 || ld < V) return ERR_BAD_SHAPE;
  logit_adjust_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, ld, row, tok, mul_pos, mul_neg, sub, n, M, V);
  return static_cast<int>(cudaGetLastError());
}

// out_tok int32 [M, k], out_lp fp32 [M, k]: the k most likely tokens per row, most likely first.
ARTB_EXPORT int artb_top_logprobs(const float* logits, long ld, const float* inv_temp, int M, int V, int k, int* out_tok,
                                  float* out_lp, cudaStream_t stream) {
  if (M <= 0 || k <= 0) return 0;
  if (V <= 0 || ld < V || k > 64) return ERR_BAD_SHAPE;
  top_logprobs_kernel<<<M, 256, 0, stream>>>(logits, ld, inv_temp, M, V, k, out_tok, out_lp);
  return static_cast<int>(cudaGetLastError());
}
