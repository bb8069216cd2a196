// Paged-KV attention for the rollout engine: cache write, decode attention over block
// tables (GQA, split-KV), and a page gather used by prefill with prefix-cache hits.
//
// Cache layout per layer: k_cache, v_cache  [num_blocks, block_size, Hkv, hd]  bf16.
// A sequence's tokens live in the blocks listed in its row of `block_table`
// [num_seqs, max_blocks]; token t is in block table[t / block_size] at offset t % block_size.
//
// Decode: one new token per sequence.  A CTA owns (sequence, kv head, split); the G = Hq/Hkv
// query heads that share the kv head form the rows of one m16 MMA tile, so K and V are read
// once for all of them.  Each of the 4 warps walks its own 32-key tiles of the split
// (cp.async into a private smem stage), keeps private online-softmax state, and the warps are
// merged through shared memory at the end.  With `splits > 1` partial (max, sum, acc) triples
// go to a workspace and a second kernel merges them.  The op is bandwidth-bound (it streams
// the KV of every running sequence once per step).
//
// This is the in-tree counterpart of the decode/prefill attention the reference delegates to
// its third-party engine (every chat.completions.create ends up there: src/art/local/vllm.py:46-53).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "bounds_check.cuh"
#include "host_utils.h"

namespace artb {

__device__ __forceinline__ void pa_cp16(void* smem, const void* gmem, bool valid) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(sz) : "memory");
}
__device__ __forceinline__ void pa_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void pa_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void pa_ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void pa_ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void pa_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pa_pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// ------------------------------------------------------------------ cache write
// qkv [M, ld] holds q | k | v columns (post-RoPE).  slot[m] = block * block_size + offset, or < 0 to skip.
__global__ void kv_write_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, int k_col, int v_col,
                                const int* __restrict__ slot, __nv_bfloat16* __restrict__ k_cache,
                                __nv_bfloat16* __restrict__ v_cache, int M, int kv_width, long num_slots, int* status) {
  const int vec = kv_width >> 3;
  const long total = static_cast<long>(M) * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int m = i / vec, c = (i % vec) * 8;
    const int s = slot[m];
    if (s < 0 || !index_ok(s, num_slots, status)) continue;
    const uint4 kv = *reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(m) * ld + k_col + c);
    const uint4 vv = *reinterpret_cast<const uint4*>(qkv + static_cast<size_t>(m) * ld + v_col + c);
    *reinterpret_cast<uint4*>(k_cache + static_cast<size_t>(s) * kv_width + c) = kv;
    *reinterpret_cast<uint4*>(v_cache + static_cast<size_t>(s) * kv_width + c) = vv;
  }
}

// Gather the first n_tok cached tokens of one sequence into contiguous k | v columns of dst [*, ld].
__global__ void kv_gather_kernel(const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                                 const int* __restrict__ block_table, int block_size, int n_tok,
                                 __nv_bfloat16* __restrict__ dst, int ld, int k_col, int v_col, int kv_width,
                                 long num_blocks, int* status) {
  const int vec = kv_width >> 3;
  const long total = static_cast<long>(n_tok) * vec;
  for (long i = blockIdx.x * static_cast<long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const int t = i / vec, c = (i % vec) * 8;
    const int blk = block_table[t / block_size];
    if (!index_ok(blk, num_blocks, status)) continue;
    const size_t s = static_cast<size_t>(blk) * block_size + t % block_size;
    *reinterpret_cast<uint4*>(dst + static_cast<size_t>(t) * ld + k_col + c) =
        *reinterpret_cast<const uint4*>(k_cache + s * kv_width + c);
    *reinterpret_cast<uint4*>(dst + static_cast<size_t>(t) * ld + v_col + c) =
        *reinterpret_cast<const uint4*>(v_cache + s * kv_width + c);
  }
}

// ------------------------------------------------------------------ decode attention
constexpr int PA_KT = 32;  // keys per warp tile

template <int HD>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, int ldq, const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table, int max_blocks,
                    const int* __restrict__ ctx_len, int block_size, int Hq, int Hkv,
                    __nv_bfloat16* __restrict__ out, int ldo, float* __restrict__ ws, int splits,
                    float scale_log2, long num_blocks, int* status) {
  constexpr int LD = HD + 8;
  extern __shared__ __align__(16) uint8_t pa_smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(pa_smem);      // [16][LD]
  __nv_bfloat16* sKV = sQ + 16 * LD;                                   // [4 warps][2 (K,V)][PA_KT][LD]
  float* sM = reinterpret_cast<float*>(sKV + 4 * 2 * PA_KT * LD);      // merge: [4][16] max, [4][16] sum
  // merge accumulators [4][16][HD] fp32: warp w's slice lives in warp w's own (by then finished) K/V staging area, which
  // keeps a CTA under a third of the SM's shared memory: three CTAs = twelve warps per SM instead of eight
  static_assert(16 * HD * 4 <= 2 * PA_KT * LD * 2, "a warp's accumulator slice must fit its K/V staging area");

  pdl_wait();                  // q, the cache rows of this step and the block table come from earlier kernels
  pdl_launch_dependents();
  const int seq = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = Hq / Hkv;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3, jm = lane >> 3, rr = lane & 7;
  const int len = ctx_len[seq];
  const int kv_width = Hkv * HD;
  const int* bt = block_table + static_cast<size_t>(seq) * max_blocks;
  const int bs_shift = (block_size & (block_size - 1)) == 0 ? 31 - __clz(block_size) : -1;   // power of two: shifts

  // Q rows: G real heads, rest zero
  for (int v = tid; v < 16 * (HD / 8); v += 128) {
    const int r = v / (HD / 8), c = (v % (HD / 8)) * 8;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (r < G) val = *reinterpret_cast<const uint4*>(q + static_cast<size_t>(seq) * ldq + (kvh * G + r) * HD + c);
    *reinterpret_cast<uint4*>(sQ + r * LD + c) = val;
  }
  __syncthreads();
  uint32_t qf[HD / 16][4];
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks)
    pa_ldsm_x4(qf[ks], sQ + ((jm & 1) * 8 + rr) * LD + ks * 16 + (jm >> 1) * 8);

  // key range of this split, in tiles of PA_KT; warps interleave tiles
  const int tiles_total = (len + PA_KT - 1) / PA_KT;
  const int tiles_per_split = (tiles_total + splits - 1) / splits;
  const int tile_lo = split * tiles_per_split;
  const int tile_hi = min(tiles_total, tile_lo + tiles_per_split);

  float acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  __nv_bfloat16* wK = sKV + warp * 2 * PA_KT * LD;
  __nv_bfloat16* wV = wK + PA_KT * LD;
  auto warp_acc = [&](int w) { return reinterpret_cast<float*>(sKV + w * 2 * PA_KT * LD); };
  for (int tile = tile_lo + warp; tile < tile_hi; tile += 4) {
    const int k0 = tile * PA_KT;
    // Warp-private load of 32 keys x HD for K and V.  A lane keeps one 16-byte column of the head and walks down the
    // rows, so the per-copy work is one table lookup and one multiply-add; with a runtime division per copy (block
    // index and offset of every key) the address arithmetic was two thirds of the kernel's instructions.
    {
      constexpr int CPR = HD / 8;                 // 16-byte copies per row
      constexpr int RPI = 32 / CPR;               // rows covered by the warp per iteration
      const int c = (lane % CPR) * 8;
      const __nv_bfloat16* kc = k_cache + kvh * HD + c;
      const __nv_bfloat16* vc = v_cache + kvh * HD + c;
#pragma unroll 4
      for (int r = lane / CPR; r < PA_KT; r += RPI) {
        const int kt = k0 + r;
        bool ok = kt < len;
        size_t s = 0;
        if (ok) {
          const int blk = bt[bs_shift >= 0 ? kt >> bs_shift : kt / block_size];
          ok = index_ok(blk, num_blocks, status);          // checked build: a bad table entry reads zeros instead
          s = static_cast<size_t>(blk) * block_size + (bs_shift >= 0 ? kt & (block_size - 1) : kt % block_size);
        }
        pa_cp16(wK + r * LD + c, kc + s * kv_width, ok);
        pa_cp16(wV + r * LD + c, vc + s * kv_width, ok);
      }
    }
    pa_commit();
    pa_wait_all();
    __syncwarp();
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) s[i][j] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int np = 0; np < 2; ++np) {
        uint32_t b[4];
        pa_ldsm_x4(b, wK + (np * 16 + (jm >> 1) * 8 + rr) * LD + ks * 16 + (jm & 1) * 8);
        pa_mma(s[np * 2], qf[ks], b[0], b[1]);
        pa_mma(s[np * 2 + 1], qf[ks], b[2], b[3]);
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int kt = k0 + i * 8 + 2 * t + j;
        float x0 = s[i][j] * scale_log2, x1 = s[i][2 + j] * scale_log2;
        if (kt >= len) x0 = x1 = -INFINITY;
        s[i][j] = x0;
        s[i][2 + j] = x1;
        mx0 = fmaxf(mx0, x0);
        mx1 = fmaxf(mx1, x1);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
    const float c0 = exp2f(m0 - ms0), c1 = exp2f(m1 - ms1);
    m0 = mn0;
    m1 = mn1;
    float rs0 = 0.f, rs1 = 0.f;
    uint32_t pf[2][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float p00 = exp2f(s[i][0] - ms0), p01 = exp2f(s[i][1] - ms0);
      const float p10 = exp2f(s[i][2] - ms1), p11 = exp2f(s[i][3] - ms1);
      rs0 += p00 + p01;
      rs1 += p10 + p11;
      pf[i >> 1][(i & 1) * 2] = pa_pack2(p00, p01);
      pf[i >> 1][(i & 1) * 2 + 1] = pa_pack2(p10, p11);
    }
    l0 = l0 * c0 + rs0;
    l1 = l1 * c1 + rs1;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      acc[i][0] *= c0;
      acc[i][1] *= c0;
      acc[i][2] *= c1;
      acc[i][3] *= c1;
    }
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
      for (int dp = 0; dp < HD / 16; ++dp) {
        uint32_t b[4];
        pa_ldsm_x4_t(b, wV + (ks * 16 + (jm & 1) * 8 + rr) * LD + dp * 16 + (jm >> 1) * 8);
        pa_mma(acc[dp * 2], pf[ks], b[0], b[1]);
        pa_mma(acc[dp * 2 + 1], pf[ks], b[2], b[3]);
      }
    }
    __syncwarp();
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  // publish per-warp state (rows g and g+8; only rows < G matter)
  if (t == 0) {
    sM[warp * 16 + g] = m0;
    sM[warp * 16 + g + 8] = m1;
    sM[64 + warp * 16 + g] = l0;
    sM[64 + warp * 16 + g + 8] = l1;
  }
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    float* a0 = warp_acc(warp) + g * HD + i * 8 + 2 * t;
    float* a1 = warp_acc(warp) + (g + 8) * HD + i * 8 + 2 * t;
    a0[0] = acc[i][0];
    a0[1] = acc[i][1];
    a1[0] = acc[i][2];
    a1[1] = acc[i][3];
  }
  __syncthreads();
  // merge the 4 warps: thread -> (row r < G, dims)
  for (int idx = tid; idx < G * HD; idx += 128) {
    const int r = idx / HD, d = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sM[w * 16 + r]);
    float lsum = 0.f, o = 0.f;
    if (mm != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float sc = exp2f(sM[w * 16 + r] - mm);
        lsum += sM[64 + w * 16 + r] * sc;
        o += warp_acc(w)[r * HD + d] * sc;
      }
    }
    const int h = kvh * G + r;
    if (splits == 1) {
      out[static_cast<size_t>(seq) * ldo + h * HD + d] = __float2bfloat16(lsum > 0.f ? o / lsum : 0.f);
    } else {
      // workspace: [seq, Hq, splits, HD + 2]
      float* w = ws + ((static_cast<size_t>(seq) * Hq + h) * splits + split) * (HD + 2);
      w[d] = o;
      if (d == 0) {
        w[HD] = mm;
        w[HD + 1] = lsum;
      }
    }
  }
}

template <int HD>
__global__ void paged_decode_merge_kernel(const float* __restrict__ ws, int splits, int Hq,
                                          __nv_bfloat16* __restrict__ out, int ldo) {
  const int seq = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const float* base = ws + (static_cast<size_t>(seq) * Hq + h) * splits * (HD + 2);
  float mm = -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, base[s * (HD + 2) + HD]);
  float lsum = 0.f, o = 0.f;
  if (mm != -INFINITY) {
    for (int s = 0; s < splits; ++s) {
      const float sc = exp2f(base[s * (HD + 2) + HD] - mm);
      lsum += base[s * (HD + 2) + HD + 1] * sc;
      o += base[s * (HD + 2) + d] * sc;
    }
  }
  out[static_cast<size_t>(seq) * ldo + h * HD + d] = __float2bfloat16(lsum > 0.f ? o / lsum : 0.f);
}

template <int HD>
static int decode_smem() {
  return (16 * (HD + 8) + 4 * 2 * PA_KT * (HD + 8)) * 2 + (2 * 4 * 16) * 4;
}

}  // namespace artb

using namespace artb;
typedef __nv_bfloat16 bf16;

ARTB_EXPORT int artb_kv_write(const void* qkv, int ld, int k_col, int v_col, const int* slot, void* k_cache,
                              void* v_cache, int M, int kv_width, long num_slots, int* status, cudaStream_t st) {
  if (M <= 0) return 0;
  if ((kv_width & 7) || (ld & 7) || (k_col & 7) || (v_col & 7)) return ERR_BAD_SHAPE;
  long total = (long)M * (kv_width / 8);
  long blocks = (total + 255) / 256;
  if (blocks > 148L * 16) blocks = 148L * 16;
  kv_write_kernel<<<(unsigned)blocks, 256, 0, st>>>((const bf16*)qkv, ld, k_col, v_col, slot, (bf16*)k_cache,
                                                   (bf16*)v_cache, M, kv_width, num_slots, status);
  return (int)cudaGetLastError();
}

ARTB_EXPORT int artb_kv_gather(const void* k_cache, const void* v_cache, const int* block_table, int block_size,
                               int n_tok, void* dst, int ld, int k_col, int v_col, int kv_width, long num_blocks,
                               int* status, cudaStream_t st) {
  if (n_tok <= 0) return 0;
  long total = (long)n_tok * (kv_width / 8);
  long blocks = (total + 255) / 256;
  if (blocks > 148L * 16) blocks = 148L * 16;
  kv_gather_kernel<<<(unsigned)blocks, 256, 0, st>>>((const bf16*)k_cache, (const bf16*)v_cache, block_table,
                                                    block_size, n_tok, (bf16*)dst, ld, k_col, v_col, kv_width,
                                                    num_blocks, status);
  return (int)cudaGetLastError();
}

// Workspace floats needed for `splits` > 1: num_seqs * Hq * splits * (hd + 2).
ARTB_EXPORT int artb_paged_decode(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                  const int* block_table, int max_blocks, const int* ctx_len, int block_size,
                                  int num_seqs, int Hq, int Hkv, int hd, void* out, int ldo, float* ws, int splits,
                                  long num_blocks, int* status, cudaStream_t st) {
  if (num_seqs <= 0) return 0;
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16 || splits < 1 || (splits > 1 && !ws)) return ERR_BAD_SHAPE;
  int dev_ = 0;
  if (cudaGetDevice(&dev_) != cudaSuccess || dev_ < 0 || dev_ >= 64) return ERR_BAD_SHAPE;
  const float scale_log2 = 1.4426950408889634f / sqrtf((float)hd);
  dim3 grid(num_seqs, Hkv, splits);
#define ARTB_PD(HD_)                                                                                             \
  {                                                                                                              \
    static bool cfgd[64] = {false};   /* the attribute is per device */                                          \
    if (!cfgd[dev_]) {                                                                                           \
      cudaFuncSetAttribute(paged_decode_kernel<HD_>, cudaFuncAttributeMaxDynamicSharedMemorySize, decode_smem<HD_>()); \
      cfgd[dev_] = true;                                                                                         \
    }                                                                                                            \
    launch_kernel(paged_decode_kernel<HD_>, grid, dim3(128), decode_smem<HD_>(), st, (const bf16*)q, ldq,        \
                  (const bf16*)k_cache, (const bf16*)v_cache, block_table, max_blocks, ctx_len, block_size, Hq, Hkv, \
                  (bf16*)out, ldo, ws, splits, scale_log2, num_blocks, status);                                  \
    if (splits > 1) paged_decode_merge_kernel<HD_><<<dim3(num_seqs, Hq), HD_, 0, st>>>(ws, splits, Hq, (bf16*)out, ldo); \
  }
  if (hd == 128) ARTB_PD(128)
  else if (hd == 64) ARTB_PD(64)
  else if (hd == 32) ARTB_PD(32)
  else return ERR_BAD_SHAPE;
#undef ARTB_PD
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------- allocation-free variant
// Split-KV decode whose workspace is a file-scope device array (see include/artb_noalloc.h for
// the contract).  In host code `g_decode_static_ws` is only a handle for the runtime: the device
// address is obtained once per device with cudaGetSymbolAddress and that pointer is what the
// kernels receive.
#include "artb_noalloc.h"

static __device__ __align__(256) float g_decode_static_ws[ARTB_DECODE_STATIC_WS_FLOATS];

static float* decode_static_ws_ptr(int* err) {
  static float* ptrs[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *err = e != cudaSuccess ? (int)e : ERR_BAD_SHAPE;
    return nullptr;
  }
  if (!ptrs[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_static_ws);   // address on the current device
    if (e != cudaSuccess) {
      *err = (int)e;
      return nullptr;
    }
    ptrs[dev] = static_cast<float*>(p);
  }
  *err = 0;
  return ptrs[dev];
}

ARTB_EXPORT int artb_paged_decode_noalloc(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                          const int* block_table, int max_blocks, const int* ctx_len, int block_size,
                                          int num_seqs, int Hq, int Hkv, int hd, void* out, int ldo, int splits,
                                          cudaStream_t st) {
  if (num_seqs <= 0) return 0;
  if (splits < 1 || hd <= 0 || Hq <= 0 || Hkv <= 0) return ERR_BAD_SHAPE;
  const long need = (long)num_seqs * Hq * splits * (hd + 2);
  if (need > (long)ARTB_DECODE_STATIC_WS_FLOATS) return ERR_TOO_LARGE;
  int err = 0;
  float* ws = decode_static_ws_ptr(&err);
  if (!ws) return err;
  return artb_paged_decode(q, ldq, k_cache, v_cache, block_table, max_blocks, ctx_len, block_size, num_seqs, Hq, Hkv,
                           hd, out, ldo, ws, splits, /*num_blocks: unknown to this entry point*/ (1L << 40), nullptr, st);
}
