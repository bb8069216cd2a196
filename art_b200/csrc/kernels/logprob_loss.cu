// Fused LM-head -> log-softmax -> selected-token log-prob -> GRPO clipped-ratio loss.
//
// Forward never materialises the [tokens, vocab] logits: the tcgen05 pipeline computes
// 128 x 256 logit tiles in TMEM and the epilogue folds each tile into per-row online
// softmax statistics (running max, running sum of exp, the logit of the target token).
// The vocabulary is split across CTAs; a token kernel merges the per-split partials,
// forms logprob = z_target - logsumexp, and evaluates
//     ratio = exp(new - old),  L = -min(ratio*A, clip(ratio, 1-eps, 1+eps_hi)*A)  (+ beta * k3 KL)
// with the per-token weight already folded with mask / normaliser, accumulating the
// loss terms and emitting dLoss/dlogprob for the backward pass.
//
// Backward recomputes the logit tiles with the same pipeline and writes
//     dlogit[t, v] = coef[t] * (onehot(target_t)[v] - exp(logit[t, v] - lse[t]))
// as bf16; a plain TN GEMM against the resident transposed LM head then gives dH.
// In a vocab-parallel (TP) layout each rank runs this over its vocabulary shard and
// the 3-float partials are what ranks exchange.
//
// Semantics restated from the reference trainer: chunked matmul + gather + logsumexp at
// src/art/local/train.py:245-281 and the loss arithmetic at src/art/local/train.py:112-151.
#include <math.h>

#include "gemm_pipeline_2cta.cuh"
#include "host_utils.h"
#include "sampling.cuh"

namespace artb {

constexpr int LP_BN = 256;
constexpr int LP_STAGES = 4;

// Work item = (m_blk, vocab split); a CTA walks the n-tiles of its split in order so the
// running statistics stay in registers.  Items with the same split are adjacent so that
// concurrently running CTAs stream the same LM-head tiles through L2.
struct SchedVocabSplit {
  int m_tiles, n_tiles, splits, tiles_per_split;
  __device__ int items_for_cta(int cta, int ncta) const {
    const int total = m_tiles * splits;
    return cta < total ? (total - cta + ncta - 1) / ncta : 0;
  }
  __device__ int tiles_for_cta(int cta, int ncta) const { return items_for_cta(cta, ncta) * tiles_per_split; }
  __device__ TileInfo get(int cta, int ncta, int i) const {
    const int item = cta + (i / tiles_per_split) * ncta;
    const int j = i % tiles_per_split;
    TileInfo ti = make_tile(item % m_tiles, 0);
    ti.group = item / m_tiles;  // split
    ti.n_blk = ti.group * tiles_per_split + j;
    ti.first = (j == 0);
    ti.last = (j == tiles_per_split - 1);
    return ti;
  }
};

struct EpiStats {
  const int* target;   // [M] target vocabulary id per row (global id, minus vocab_offset locally)
  float* partials;     // [splits, M, 4]  (max, sumexp, z_target, unused)
  int M, V, vocab_offset;
  float run_max, run_sum, z;
  int tgt;

  __device__ void tile_begin(const TileInfo& ti, int row) {
    if (ti.first) {
      run_max = -INFINITY;
      run_sum = 0.f;
      z = -INFINITY;
      const int gr = ti.m_blk * GEMM_BM + row;
      tgt = (gr < M) ? target[gr] - vocab_offset : -1;
    }
  }
  __device__ void chunk(const TileInfo& ti, int row, int c, uint32_t (&acc)[32]) {
    const int gc = ti.n_blk * LP_BN + c;
    if (gc >= V) return;
    float cmax = -INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float v = __uint_as_float(acc[j]);
      if (gc + j >= V) v = -INFINITY;
      acc[j] = __float_as_uint(v);
      cmax = fmaxf(cmax, v);
    }
    const float nmax = fmaxf(run_max, cmax);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) s += __expf(__uint_as_float(acc[j]) - nmax);
    run_sum = run_sum * __expf(run_max - nmax) + s;
    run_max = nmax;
    const int d = tgt - gc;
    if (d >= 0 && d < 32) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j == d) z = __uint_as_float(acc[j]);
    }
  }
  __device__ void tile_end(const TileInfo& ti, int row) {
    if (!ti.last) return;
    const int gr = ti.m_blk * GEMM_BM + row;
    if (gr >= M) return;
    float4 o = make_float4(run_max, run_sum, z, 0.f);
    *reinterpret_cast<float4*>(partials + (static_cast<size_t>(ti.group) * M + gr) * 4) = o;
  }
};

struct EpiDLogits {
  const int* target;
  const float* lse;    // [M]
  const float* coef;   // [M] dLoss/dlogprob
  __nv_bfloat16* out;  // [M, ldo]
  int M, V, ldo, vocab_offset;
  float my_lse, my_coef;
  int tgt;

  __device__ void tile_begin(const TileInfo& ti, int row) {
    const int gr = ti.m_blk * GEMM_BM + row;
    if (gr < M) {
      my_lse = lse[gr];
      my_coef = coef[gr];
      tgt = target[gr] - vocab_offset;
    } else {
      my_lse = 0.f;
      my_coef = 0.f;
      tgt = -1;
    }
  }
  __device__ void chunk(const TileInfo& ti, int row, int c, uint32_t (&acc)[32]) {
    const int gr = ti.m_blk * GEMM_BM + row;
    const int gc = ti.n_blk * LP_BN + c;
    if (gr >= M || gc >= ldo) return;
    __nv_bfloat16* o = out + static_cast<size_t>(gr) * ldo + gc;
    uint32_t packed[16];
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      float p0 = __expf(__uint_as_float(acc[j]) - my_lse);
      float p1 = __expf(__uint_as_float(acc[j + 1]) - my_lse);
      float d0 = my_coef * (((gc + j) == tgt ? 1.f : 0.f) - p0);
      float d1 = my_coef * (((gc + j + 1) == tgt ? 1.f : 0.f) - p1);
      if (gc + j >= V) d0 = 0.f;
      if (gc + j + 1 >= V) d1 = 0.f;
      packed[j >> 1] = pack_bf16x2(d0, d1);
    }
    if (gc + 32 <= ldo) {
#pragma unroll
      for (int j = 0; j < 16; j += 4)
        *reinterpret_cast<uint4*>(o + 2 * j) = make_uint4(packed[j], packed[j + 1], packed[j + 2], packed[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (gc + 2 * j + 1 < ldo) *reinterpret_cast<uint32_t*>(o + 2 * j) = packed[j];
    }
  }
  __device__ void tile_end(const TileInfo&, int) {}
};

// Sampling epilogue for the rollout engine: temperature-scaled online softmax statistics plus a
// running Gumbel-max argmax, so one pass over the LM head yields the sampled token and its
// log-probability under the sampling distribution without materialising logits.
//   x = logit * inv_temp ;  sample = argmax_v (x_v + g_v),  g_v = -log(-log(u_v)),  u_v = hash(seed, row, v)
// inv_temp == 0 selects greedy decoding (argmax of the raw logits, log-prob at temperature 1).
struct EpiSample {
  float* partials;        // [splits, M, 8]: max, sumexp, best_score, best_idx(bits), best_x, -, -, -
  const float* inv_temp;  // [M] per-row 1/temperature (0 = greedy)
  const uint32_t* row_seed;  // [M] per-row seed (request seed mixed with the decode step)
  int M, V, vocab_offset;
  float run_max, run_sum, best_score, best_x, it;
  int best_idx;
  uint32_t seed;

  __device__ void tile_begin(const TileInfo& ti, int row) {
    if (ti.first) {
      run_max = -INFINITY;
      run_sum = 0.f;
      best_score = -INFINITY;
      best_x = 0.f;
      best_idx = -1;
      const int gr = ti.m_blk * GEMM_BM + row;
      it = (gr < M) ? inv_temp[gr] : 0.f;
      seed = (gr < M) ? row_seed[gr] : 0u;
    }
  }
  __device__ void chunk(const TileInfo& ti, int row, int c, uint32_t (&acc)[32]) {
    const int gc = ti.n_blk * LP_BN + c;
    if (gc >= V) return;
    const uint32_t gr = ti.m_blk * GEMM_BM + row;
    const bool greedy = it == 0.f;
    const float sc = greedy ? 1.f : it;
    float cmax = -INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float x = __uint_as_float(acc[j]) * sc;
      if (gc + j >= V) x = -INFINITY;
      acc[j] = __float_as_uint(x);
      cmax = fmaxf(cmax, x);
    }
    const float nmax = fmaxf(run_max, cmax);
    float ssum = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float x = __uint_as_float(acc[j]);
      ssum += __expf(x - nmax);
      float score = x;
      if (!greedy) score += gumbel_noise(seed, gr, static_cast<uint32_t>(vocab_offset + gc + j));
      if (score > best_score) {
        best_score = score;
        best_x = x;
        best_idx = vocab_offset + gc + j;
      }
    }
    run_sum = run_sum * __expf(run_max - nmax) + ssum;
    run_max = nmax;
  }
  __device__ void tile_end(const TileInfo& ti, int row) {
    if (!ti.last) return;
    const int gr = ti.m_blk * GEMM_BM + row;
    if (gr >= M) return;
    float* o = partials + (static_cast<size_t>(ti.group) * M + gr) * 8;
    *reinterpret_cast<float4*>(o) = make_float4(run_max, run_sum, best_score, __int_as_float(best_idx));
    *reinterpret_cast<float4*>(o + 4) = make_float4(best_x, 0.f, 0.f, 0.f);
  }
};

// Merge sampling partials (over vocabulary splits and, for tensor-parallel heads, over ranks'
// partial buffers laid out back to back): token id and log-prob per row.
__global__ void sample_merge_kernel(const float* __restrict__ partials, int parts, int M, int* __restrict__ token,
                                    float* __restrict__ logprob) {
  const int tI = blockIdx.x * blockDim.x + threadIdx.x;
  if (tI >= M) return;
  float mx = -INFINITY;
  for (int s = 0; s < parts; ++s) mx = fmaxf(mx, partials[(static_cast<size_t>(s) * M + tI) * 8]);
  float sum = 0.f, best = -INFINITY, bx = 0.f;
  int bi = -1;
  for (int s = 0; s < parts; ++s) {
    const float* p = partials + (static_cast<size_t>(s) * M + tI) * 8;
    sum += p[1] * __expf(p[0] - mx);
    if (p[2] > best) {
      best = p[2];
      bi = __float_as_int(p[3]);
      bx = p[4];
    }
  }
  token[tI] = bi;
  logprob[tI] = bx - (mx + logf(sum));
}

// Merge vocabulary-split partials and evaluate the per-token GRPO terms.
//   partials [splits, M, 4];  old_lp may hold NaN (= "sampled under the current policy");
//   tok_w = weight * mask / normaliser (already shifted to next-token alignment);
//   accum[0] += sum(pg * tok_w), accum[1] += sum(kl * tok_w), accum[2] += sum(tok_w > 0)
__global__ void grpo_token_kernel(const float* __restrict__ partials, int splits, int M,
                                  const float* __restrict__ old_lp, const float* __restrict__ adv,
                                  const float* __restrict__ tok_w, const float* __restrict__ ref_lp,
                                  float eps_lo, float eps_hi, float beta, float* __restrict__ lse_out,
                                  float* __restrict__ lp_out, float* __restrict__ coef_out,
                                  float* __restrict__ accum) {
  float loc_pg = 0.f, loc_kl = 0.f, loc_n = 0.f;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < M; t += gridDim.x * blockDim.x) {
    float mx = -INFINITY;
    for (int s = 0; s < splits; ++s) mx = fmaxf(mx, partials[(static_cast<size_t>(s) * M + t) * 4]);
    float sum = 0.f, z = -INFINITY;
    for (int s = 0; s < splits; ++s) {
      const float* p = partials + (static_cast<size_t>(s) * M + t) * 4;
      sum += p[1] * __expf(p[0] - mx);
      z = fmaxf(z, p[2]);
    }
    const float lse = mx + logf(sum);
    const float lp = z - lse;
    lse_out[t] = lse;
    lp_out[t] = lp;
    float c = 0.f;
    if (tok_w) {
      const float w = tok_w[t];
      if (w != 0.f) {
        float old = old_lp[t];
        if (isnan(old)) old = lp;
        const float a = adv[t];
        const float ratio = expf(lp - old);
        const float unclipped = ratio * a;
        const float clipped = fminf(fmaxf(ratio, 1.f - eps_lo), 1.f + eps_hi) * a;
        const float pg = -fminf(unclipped, clipped);
        const bool inside = (ratio >= 1.f - eps_lo) && (ratio <= 1.f + eps_hi);
        float dpg_dlp = (inside || unclipped < clipped) ? -a * ratio : 0.f;
        float kl = 0.f, dkl_dlp = 0.f;
        if (ref_lp && beta > 0.f) {
          const float d = ref_lp[t] - lp;
          const float e = expf(d);
          kl = e - d - 1.f;
          dkl_dlp = 1.f - e;
        }
        loc_pg += pg * w;
        loc_kl += kl * w;
        loc_n += 1.f;
        c = w * (dpg_dlp + beta * dkl_dlp);
      }
    }
    if (coef_out) coef_out[t] = c;
  }
  // block reduce
  __shared__ float red[3][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    loc_pg += __shfl_xor_sync(0xffffffffu, loc_pg, o);
    loc_kl += __shfl_xor_sync(0xffffffffu, loc_kl, o);
    loc_n += __shfl_xor_sync(0xffffffffu, loc_n, o);
  }
  if (lane == 0) {
    red[0][warp] = loc_pg;
    red[1][warp] = loc_kl;
    red[2][warp] = loc_n;
  }
  __syncthreads();
  if (warp == 0 && accum) {
    const int nw = blockDim.x >> 5;
    float a = lane < nw ? red[0][lane] : 0.f, b = lane < nw ? red[1][lane] : 0.f, c = lane < nw ? red[2][lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, o);
      b += __shfl_xor_sync(0xffffffffu, b, o);
      c += __shfl_xor_sync(0xffffffffu, c, o);
    }
    if (lane == 0) {
      atomicAdd(accum + 0, a);
      atomicAdd(accum + 1, b);
      atomicAdd(accum + 2, c);
    }
  }
}

// From this many token rows on, the LM-head kernels run on CTA pairs (256 x 256 logit tiles, the pair shares each
// LM-head tile in shared memory); below it (decode batches) one CTA per 128 x 256 tile fills the machine better.
static bool lp_pairs(int M) { return M >= 4 * GEMM_BM; }

template <class Epi>
static int launch_lp(const void* H, int ldh, const void* W, int ldw, int M, int V, int K, int splits,
                     const Epi& epi, int* status, cudaStream_t stream) {
  CUtensorMap tA, tB;
  int e;
  int dev = 0;
  cudaGetDevice(&dev);
  SchedVocabSplit sched;
  sched.n_tiles = (V + LP_BN - 1) / LP_BN;
  sched.splits = splits;
  sched.tiles_per_split = (sched.n_tiles + splits - 1) / splits;
  const int kb = (K + GEMM_BK - 1) / GEMM_BK;
  if ((e = make_tmap_bf16_2d(&tA, H, M, K, ldh, GEMM_BM, GEMM_BK))) return e;
  if (lp_pairs(M)) {
    using L = Gemm2SmemLayout<6, LP_BN>;
    auto kern = gemm_tcgen05_2cta_kernel<6, LP_BN, SchedVocabSplit, Epi>;
    static bool configured[64] = {false};
    if (!configured[dev & 63]) {
      cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
      if (ce != cudaSuccess) return static_cast<int>(ce);
      configured[dev & 63] = true;
    }
    if ((e = make_tmap_bf16_2d(&tB, W, V, K, ldw, LP_BN / 2, GEMM_BK))) return e;
    sched.m_tiles = (M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);      // pair tiles of 256 rows
    int clusters = sched.m_tiles * splits;
    if (clusters > sm_count() / 2) clusters = sm_count() / 2;
    return static_cast<int>(launch_kernel(kern, dim3(2 * clusters), dim3(gemm_pipe_threads<Epi>()), L::TOTAL, stream, tA, tB,
                                          tA, tB, kb, 0, sched, epi, status, NoComm{}));
  }
  using L = GemmSmemLayout<LP_BN, LP_STAGES>;
  auto kern = gemm_tcgen05_kernel<LP_BN, LP_STAGES, SchedVocabSplit, Epi>;
  static bool configured[64] = {false};
  if (!configured[dev & 63]) {
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (ce != cudaSuccess) return static_cast<int>(ce);
    configured[dev & 63] = true;
  }
  if ((e = make_tmap_bf16_2d(&tB, W, V, K, ldw, LP_BN, GEMM_BK))) return e;
  sched.m_tiles = (M + GEMM_BM - 1) / GEMM_BM;
  int grid = sched.m_tiles * splits;
  if (grid > sm_count()) grid = sm_count();
  return static_cast<int>(launch_kernel(kern, dim3(grid), dim3(gemm_pipe_threads<Epi>()), L::TOTAL, stream, tA, tB, tA, tB, kb,
                                        0, sched, epi, status, NoComm{}));
}

}  // namespace artb

using namespace artb;

// Number of vocabulary splits the forward uses for (M, V): enough (m_blk, split) items to
// fill the machine, never more splits than n-tiles.  The partials buffer is [splits, M, 4] fp32.
ARTB_EXPORT int artb_logprob_splits(int M, int V) {
  const bool pairs = lp_pairs(M);
  const int m_tiles = pairs ? (M + 2 * GEMM_BM - 1) / (2 * GEMM_BM) : (M + GEMM_BM - 1) / GEMM_BM;
  const int n_tiles = (V + LP_BN - 1) / LP_BN;
  const int workers = pairs ? sm_count() / 2 : sm_count();
  int splits = (2 * workers + m_tiles - 1) / m_tiles;
  if (splits < 1) splits = 1;
  if (splits > n_tiles) splits = n_tiles;
  // make the last split non-empty
  while (splits > 1 && ((n_tiles + splits - 1) / splits) * (splits - 1) >= n_tiles) --splits;
  return splits;
}

// Phase 1: per-split online-softmax partials over the vocabulary shard W[V, K].
ARTB_EXPORT int artb_logprob_partials(const void* H, int ldh, const void* W, int ldw, const int* target,
                                      float* partials, int M, int V, int K, int splits, int vocab_offset,
                                      int* status, cudaStream_t stream) {
  if (M <= 0 || V <= 0 || (K & 7)) return ERR_BAD_SHAPE;
  EpiStats epi;
  epi.target = target;
  epi.partials = partials;
  epi.M = M;
  epi.V = V;
  epi.vocab_offset = vocab_offset;
  epi.run_max = 0.f;
  epi.run_sum = 0.f;
  epi.z = 0.f;
  epi.tgt = -1;
  return launch_lp(H, ldh, W, ldw, M, V, K, splits, epi, status, stream);
}

// Phase 2: merge partials -> lse, logprob; GRPO terms; coef = dLoss/dlogprob.
// tok_w == nullptr: only lse/logprob are produced (reference-policy pass).
ARTB_EXPORT int artb_grpo_tokens(const float* partials, int splits, int M, const float* old_lp, const float* adv,
                                 const float* tok_w, const float* ref_lp, float eps_lo, float eps_hi, float beta,
                                 float* lse, float* lp, float* coef, float* accum, cudaStream_t stream) {
  if (M <= 0) return 0;
  int grid = (M + 255) / 256;
  if (grid > 1024) grid = 1024;
  grpo_token_kernel<<<grid, 256, 0, stream>>>(partials, splits, M, old_lp, adv, tok_w, ref_lp, eps_lo, eps_hi, beta,
                                              lse, lp, coef, accum);
  return static_cast<int>(cudaGetLastError());
}

// Backward phase 1: dlogits[M, ldo] (bf16) by recomputation.  ldo >= V, multiple of 8;
// columns V..ldo-1 are written as zero.
ARTB_EXPORT int artb_logprob_dlogits(const void* H, int ldh, const void* W, int ldw, const int* target,
                                     const float* lse, const float* coef, void* dlogits, int ldo, int M, int V,
                                     int K, int vocab_offset, int* status, cudaStream_t stream) {
  if (M <= 0 || V <= 0 || (K & 7) || (ldo & 7) || ldo < V) return ERR_BAD_SHAPE;
  EpiDLogits epi;
  epi.target = target;
  epi.lse = lse;
  epi.coef = coef;
  epi.out = reinterpret_cast<__nv_bfloat16*>(dlogits);
  epi.M = M;
  epi.V = V;
  epi.ldo = ldo;
  epi.vocab_offset = vocab_offset;
  epi.my_lse = 0.f;
  epi.my_coef = 0.f;
  epi.tgt = -1;
  // one split per n-tile group is irrelevant here (no cross-tile state): reuse the
  // vocab-split schedule so LM-head tiles are shared through L2 the same way.
  int splits = artb_logprob_splits(M, V);
  return launch_lp(H, ldh, W, ldw, M, V, K, splits, epi, status, stream);
}

// Rollout sampling: partials [splits, M, 8] for one vocabulary shard (see EpiSample).
ARTB_EXPORT int artb_sample_partials(const void* H, int ldh, const void* W, int ldw, const float* inv_temp,
                                     const uint32_t* row_seed, float* partials, int M, int V, int K, int splits,
                                     int vocab_offset, int* status, cudaStream_t stream) {
  if (M <= 0 || V <= 0 || (K & 7)) return ERR_BAD_SHAPE;
  EpiSample epi;
  epi.partials = partials;
  epi.inv_temp = inv_temp;
  epi.row_seed = row_seed;
  epi.M = M;
  epi.V = V;
  epi.vocab_offset = vocab_offset;
  epi.run_max = epi.run_sum = epi.best_score = epi.best_x = epi.it = 0.f;
  epi.best_idx = -1;
  epi.seed = 0;
  return launch_lp(H, ldh, W, ldw, M, V, K, splits, epi, status, stream);
}

ARTB_EXPORT int artb_sample_merge(const float* partials, int parts, int M, int* token, float* logprob,
                                  cudaStream_t stream) {
  if (M <= 0) return 0;
  sample_merge_kernel<<<(M + 127) / 128, 128, 0, stream>>>(partials, parts, M, token, logprob);
  return static_cast<int>(cudaGetLastError());
}
