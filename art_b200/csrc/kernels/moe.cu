// Mixture-of-experts routing kernels: softmax/top-k router, expert-sorted row plan, row
// gather (dispatch on one GPU), weighted combine, and the router's backward.
//
//   router   logits[M, E] -> top-k expert ids and weights per token (+ per-expert counts)
//   plan     counts -> segment offsets padded to 128 rows, tile -> expert map for the grouped GEMM
//   assign   (token, slot) -> row position inside its expert's segment
//   gather   xp[pos] = scale * x[token]                       (rows sorted by expert)
//   combine  out[token] = residual[token] + sum_slot w * yp[pos(token, slot)]   (fixed order)
//   router_bwd  d(top-k weights) -> d(logits)
//
// The reference supports dense models only; these serve the sparse-expert configuration
// (128 experts, top-8).  Unfused equivalent: torch.topk + index_select / index_add_.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "host_utils.h"

namespace artb {

constexpr int MOE_MAX_E_PER_LANE = 8;   // up to 256 experts
constexpr int MOE_MAX_K = 16;

// Element `e` of a per-lane-strided register array (entry e lives in lane e % 32, slot e / 32),
// broadcast to the whole warp.  `e` must be warp-uniform.  Select chain keeps the array in registers.
__device__ __forceinline__ float warp_pick(const float (&a)[MOE_MAX_E_PER_LANE], int e) {
  float v = a[0];
#pragma unroll
  for (int j = 1; j < MOE_MAX_E_PER_LANE; ++j)
    if (j == (e >> 5)) v = a[j];
  return __shfl_sync(0xffffffffu, v, e & 31);
}

// One warp per token.
__global__ void moe_router_kernel(const float* __restrict__ logits, int ld, int M, int E, int k, int norm,
                                  int* __restrict__ topi, float* __restrict__ topw, int* __restrict__ counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= M) return;
  const float* row = logits + static_cast<size_t>(warp) * ld;
  float v[MOE_MAX_E_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MOE_MAX_E_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    v[j] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < MOE_MAX_E_PER_LANE; ++j) {
    v[j] = (j * 32 + lane) < E ? __expf(v[j] - mx) : -1.f;   // probabilities are >= 0; -1 marks "taken / absent"
    if (v[j] > 0.f) sum += v[j];
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  float wsel = 0.f, wtot = 0.f;
  int isel = 0;
  for (int s = 0; s < k; ++s) {
    float best = -2.f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MOE_MAX_E_PER_LANE; ++j)
      if (v[j] > best) {
        best = v[j];
        bi = j * 32 + lane;
      }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
#pragma unroll
    for (int j = 0; j < MOE_MAX_E_PER_LANE; ++j)
      if (j == (bi >> 5) && (bi & 31) == lane) v[j] = -1.f;
    const float p = best * inv;
    wtot += p;
    if (lane == s) {
      wsel = p;
      isel = bi;
    }
  }
  if (lane < k) {
    topi[static_cast<size_t>(warp) * k + lane] = isel;
    topw[static_cast<size_t>(warp) * k + lane] = norm ? wsel / wtot : wsel;
    atomicAdd(counts + isel, 1);
  }
}

// Single block.  seg_off[E+1]: padded exclusive offsets; tile_expert[cap_tiles]; cursor[E] = 0.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int E, int* __restrict__ seg_off,
                                int* __restrict__ tile_expert, int cap_tiles, int* __restrict__ cursor) {
  __shared__ int s_off[257];
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = off;
      off += (counts[e] + 127) / 128 * 128;
    }
    s_off[E] = off;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) seg_off[e] = s_off[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) cursor[e] = 0;
  for (int t = threadIdx.x; t < cap_tiles; t += blockDim.x) {
    const int row = t * 128;
    int ex = -1;
    if (row < s_off[E]) {
      int lo = 0, hi = E;   // last e with s_off[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_off[mid] <= row) lo = mid;
        else hi = mid;
      }
      ex = lo;
    }
    tile_expert[t] = ex;
  }
}

__global__ void moe_fill_kernel(int* __restrict__ row_token, float* __restrict__ row_w, long n) {
  const long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  if (i < n) {
    row_token[i] = -1;
    row_w[i] = 0.f;
  }
}

__global__ void moe_assign_kernel(const int* __restrict__ topi, const float* __restrict__ topw, long n /* M*k */, int k,
                                  const int* __restrict__ seg_off, int* __restrict__ cursor, int* __restrict__ pos,
                                  int* __restrict__ row_token, float* __restrict__ row_w) {
  const long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const int e = topi[i];
  const int p = seg_off[e] + atomicAdd(cursor + e, 1);
  pos[i] = p;
  row_token[p] = static_cast<int>(i / k);
  row_w[p] = topw[i];
}

// xp[r] = (use_w ? row_w[r] : 1) * x[row_token[r]], zeros for padding rows; rows >= seg_off[E] untouched.
__global__ void __launch_bounds__(128)
moe_gather_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int* __restrict__ row_token,
                  const float* __restrict__ row_w, int use_w, const int* __restrict__ total_rows,
                  __nv_bfloat16* __restrict__ xp, int ldp, int D) {
  const int r = blockIdx.x;
  if (r >= *total_rows) return;
  const int t = row_token[r];
  uint4* dst = reinterpret_cast<uint4*>(xp + static_cast<size_t>(r) * ldp);
  const int nv = D >> 3;
  if (t < 0) {
    for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * ldx);
  const float w = use_w ? row_w[r] : 1.f;
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

// out[t] = residual[t] + sum_s w[t,s] * yp[pos[t,s]]  (w == nullptr: plain sum);
// optional dots[t,s] = <g[t], yp[pos[t,s]]> (gradient of the routing weight).
__global__ void __launch_bounds__(128)
moe_combine_kernel(const __nv_bfloat16* __restrict__ yp, int ldp, const int* __restrict__ pos,
                   const float* __restrict__ w, int k, const __nv_bfloat16* __restrict__ residual, int ldr,
                   __nv_bfloat16* __restrict__ out, int ldo, int D, const __nv_bfloat16* __restrict__ g, int ldg,
                   float* __restrict__ dots) {
  const int t = blockIdx.x;
  __shared__ int s_pos[MOE_MAX_K];
  __shared__ float s_w[MOE_MAX_K];
  __shared__ float s_dot[MOE_MAX_K][4];
  if (threadIdx.x < k) {
    s_pos[threadIdx.x] = pos[static_cast<size_t>(t) * k + threadIdx.x];
    s_w[threadIdx.x] = w ? w[static_cast<size_t>(t) * k + threadIdx.x] : 1.f;
  }
  __syncthreads();
  float dot[MOE_MAX_K];
#pragma unroll
  for (int s = 0; s < MOE_MAX_K; ++s) dot[s] = 0.f;
  const int nv = D >> 3;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float acc[8];
    if (residual) {
      const uint4 rv = reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * ldr)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    float gv[8];
    if (dots) {
      const uint4 rv = reinterpret_cast<const uint4*>(g + static_cast<size_t>(t) * ldg)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        gv[2 * j] = f.x;
        gv[2 * j + 1] = f.y;
      }
    }
#pragma unroll
    for (int s = 0; s < MOE_MAX_K; ++s) {
      if (s < k) {
        const uint4 yv = reinterpret_cast<const uint4*>(yp + static_cast<size_t>(s_pos[s]) * ldp)[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&yv);
        const float ws = s_w[s];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float2 f = __bfloat1622float2(h[j]);
          acc[2 * j] += ws * f.x;
          acc[2 * j + 1] += ws * f.y;
          if (dots) dot[s] += gv[2 * j] * f.x + gv[2 * j + 1] * f.y;
        }
      }
    }
    if (out) {
      uint4 ov;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
      reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * ldo)[i] = ov;
    }
  }
  if (dots) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int s = 0; s < MOE_MAX_K; ++s) {
      if (s < k) {
        float d = dot[s];
#pragma unroll
        for (int o = 16; o; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        if (lane == 0) s_dot[s][warp] = d;
      }
    }
    __syncthreads();
    if (threadIdx.x < k)
      dots[static_cast<size_t>(t) * k + threadIdx.x] =
          s_dot[threadIdx.x][0] + s_dot[threadIdx.x][1] + s_dot[threadIdx.x][2] + s_dot[threadIdx.x][3];
  }
}

// d(logits) from d(top-k weights).  p = softmax(logits); w_s = p_s / Z (Z = sum of selected p, or 1).
//   dp_s = (dw_s - sum_j dw_j w_j) / Z   (norm)   |   dp_s = dw_s   (no norm);  dp = 0 for unselected
//   dlogit_e = p_e * (dp_e - sum_j dp_j p_j)
__global__ void moe_router_bwd_kernel(const float* __restrict__ logits, int ld, const int* __restrict__ topi,
                                      const float* __restrict__ topw, const float* __restrict__ dw, int M, int E, int k,
                                      int norm, __nv_bfloat16* __restrict__ dlogits, int ldd) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= M) return;
  const float* row = logits + static_cast<size_t>(warp) * ld;
  float p[MOE_MAX_E_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < MOE_MAX_E_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    p[j] = e < E ? row[e] : -INFINITY;
    mx = fmaxf(mx, p[j]);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < MOE_MAX_E_PER_LANE; ++j) {
    p[j] = (j * 32 + lane) < E ? __expf(p[j] - mx) : 0.f;
    sum += p[j];
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  // selected entries live in lanes 0..k-1
  int ie = 0;
  float w = 0.f, g = 0.f;
  if (lane < k) {
    ie = topi[static_cast<size_t>(warp) * k + lane];
    w = topw[static_cast<size_t>(warp) * k + lane];
    g = dw[static_cast<size_t>(warp) * k + lane];
  }
  float dp = g;
  if (norm) {
    float gw = g * w;
#pragma unroll
    for (int o = 16; o; o >>= 1) gw += __shfl_xor_sync(0xffffffffu, gw, o);
    // Z = p_sel / w  (any selected entry); take it from lane 0
    const int e0 = __shfl_sync(0xffffffffu, ie, 0);
    const float w0 = __shfl_sync(0xffffffffu, w, 0);
    const float p0 = warp_pick(p, e0) * inv;
    const float Z = p0 / fmaxf(w0, 1e-20f);
    dp = (g - gw) / Z;
  }
  // sum_j dp_j p_j over the selected entries
  float pe = 0.f;
  float dpp = 0.f;
  {
    // fetch p of my selected expert from its owner lane
    float psel = 0.f;
    for (int s = 0; s < k; ++s) {
      const int es = __shfl_sync(0xffffffffu, ie, s);
      const float v = warp_pick(p, es) * inv;
      if (lane == s) psel = v;
    }
    pe = psel;
    dpp = lane < k ? dp * pe : 0.f;
#pragma unroll
    for (int o = 16; o; o >>= 1) dpp += __shfl_xor_sync(0xffffffffu, dpp, o);
  }
  __nv_bfloat16* out = dlogits + static_cast<size_t>(warp) * ldd;
#pragma unroll
  for (int j = 0; j < MOE_MAX_E_PER_LANE; ++j) {
    const int e = j * 32 + lane;
    if (e < ldd) out[e] = __float2bfloat16(e < E ? p[j] * inv * (0.f - dpp) : 0.f);
  }
  __syncwarp();
  if (lane < k) out[ie] = __float2bfloat16(pe * (dp - dpp));
}

}  // namespace artb

using namespace artb;

// logits fp32 [M, E] (E <= 256, k <= 16); counts int32 [E] must be zero on entry.
ARTB_EXPORT int artb_moe_router(const float* logits, int ld, int M, int E, int k, int norm, int* topi, float* topw,
                                int* counts, cudaStream_t st) {
  if (M <= 0) return 0;
  if (E <= 0 || E > 32 * MOE_MAX_E_PER_LANE || k <= 0 || k > MOE_MAX_K || k > E) return ERR_BAD_SHAPE;
  const int threads = 256, warps = threads / 32;
  moe_router_kernel<<<(M + warps - 1) / warps, threads, 0, st>>>(logits, ld, M, E, k, norm, topi, topw, counts);
  return static_cast<int>(cudaGetLastError());
}

// seg_off int32 [E+1], tile_expert int32 [cap_tiles], cursor int32 [E], pos int32 [M*k],
// row_token int32 [cap_tiles*128], row_w fp32 [cap_tiles*128].
ARTB_EXPORT int artb_moe_plan(const int* counts, int E, const int* topi, const float* topw, long M, int k, int* seg_off,
                              int* tile_expert, int cap_tiles, int* cursor, int* pos, int* row_token, float* row_w,
                              cudaStream_t st) {
  if (E <= 0 || E > 256 || cap_tiles <= 0) return ERR_BAD_SHAPE;
  if (static_cast<long>(cap_tiles) * 128 < M * k + static_cast<long>(E) * 127) return ERR_TOO_LARGE;
  moe_plan_kernel<<<1, 256, 0, st>>>(counts, E, seg_off, tile_expert, cap_tiles, cursor);
  const long rows = static_cast<long>(cap_tiles) * 128;
  moe_fill_kernel<<<static_cast<unsigned>((rows + 255) / 256), 256, 0, st>>>(row_token, row_w, rows);
  const long n = M * k;
  if (n > 0)
    moe_assign_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(topi, topw, n, k, seg_off, cursor, pos,
                                                                              row_token, row_w);
  return static_cast<int>(cudaGetLastError());
}

ARTB_EXPORT int artb_moe_gather(const void* x, int ldx, const int* row_token, const float* row_w, int use_w,
                                const int* total_rows, void* xp, int ldp, int D, int cap_rows, cudaStream_t st) {
  if (cap_rows <= 0) return 0;
  if ((D & 7) || (ldx & 7) || (ldp & 7)) return ERR_BAD_SHAPE;
  moe_gather_kernel<<<cap_rows, 128, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx, row_token, row_w, use_w,
                                             total_rows, reinterpret_cast<__nv_bfloat16*>(xp), ldp, D);
  return static_cast<int>(cudaGetLastError());
}

ARTB_EXPORT int artb_moe_combine(const void* yp, int ldp, const int* pos, const float* w, int M, int k,
                                 const void* residual, int ldr, void* out, int ldo, int D, const void* g, int ldg,
                                 float* dots, cudaStream_t st) {
  if (M <= 0) return 0;
  if ((D & 7) || (ldp & 7) || k > MOE_MAX_K) return ERR_BAD_SHAPE;
  moe_combine_kernel<<<M, 128, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(yp), ldp, pos, w, k,
                                        reinterpret_cast<const __nv_bfloat16*>(residual), ldr,
                                        reinterpret_cast<__nv_bfloat16*>(out), ldo, D,
                                        reinterpret_cast<const __nv_bfloat16*>(g), ldg, dots);
  return static_cast<int>(cudaGetLastError());
}

ARTB_EXPORT int artb_moe_router_bwd(const float* logits, int ld, const int* topi, const float* topw, const float* dw,
                                    int M, int E, int k, int norm, void* dlogits, int ldd, cudaStream_t st) {
  if (M <= 0) return 0;
  if (E > 32 * MOE_MAX_E_PER_LANE || k > MOE_MAX_K || ldd < E || ldd > 32 * MOE_MAX_E_PER_LANE) return ERR_BAD_SHAPE;
  const int threads = 256, warps = threads / 32;
  moe_router_bwd_kernel<<<(M + warps - 1) / warps, threads, 0, st>>>(
      logits, ld, topi, topw, dw, M, E, k, norm, reinterpret_cast<__nv_bfloat16*>(dlogits), ldd);
  return static_cast<int>(cudaGetLastError());
}
