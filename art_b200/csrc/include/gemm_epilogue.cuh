// Tile schedules and the store epilogue shared by the dense GEMM entry points.
#pragma once
#include "gemm_pipeline.cuh"

namespace artb {

enum GemmEpilogue : int { EPI_BF16 = 0, EPI_BF16_RESID = 1, EPI_F32 = 2, EPI_SWIGLU = 3, EPI_SWIGLU_BWD = 4 };

// Tiles are visited with the M index fastest inside bands of group_m tile rows (see raster_tile), so the CTAs that
// run concurrently share a band of the activation matrix that stays L2-resident and a handful of weight (B) tiles.
struct SchedMFast {
  int m_tiles, n_tiles, group_m;
  __device__ int tiles_for_cta(int cta, int ncta) const {
    const int total = m_tiles * n_tiles;
    return cta < total ? (total - cta + ncta - 1) / ncta : 0;
  }
  __device__ TileInfo get(int cta, int ncta, int i) const {
    int m, n;
    raster_tile(cta + i * ncta, m_tiles, n_tiles, group_m, m, n);
    return make_tile(m, n);
  }
};

// Tile rows per band so that a band of A (rows x K bf16) is about 28 MB: small enough to stay in the 126 MB L2 next to
// the streaming B and C traffic, large enough that B is re-read only a few times.
inline int pick_group_m(int m_tiles, int tile_rows, int K) {
  long g = (28L << 20) / (static_cast<long>(tile_rows) * K * 2);
  if (g < 4) g = 4;
  if (g > m_tiles) g = m_tiles;
  return static_cast<int>(g);
}

// Split-K schedule for small-M (decode) GEMMs: work item = (m_blk, n_blk, k_split); every item
// covers kb_per K blocks of the main operand, the extra-K operand goes with split 0.
struct SchedSplitK {
  int m_tiles, n_tiles, splits, kb_per, kb_main;
  __device__ int tiles_for_cta(int cta, int ncta) const {
    const int total = m_tiles * n_tiles * splits;
    return cta < total ? (total - cta + ncta - 1) / ncta : 0;
  }
  __device__ TileInfo get(int cta, int ncta, int i) const {
    const int t = cta + i * ncta;
    TileInfo ti = make_tile(t % m_tiles, (t / m_tiles) % n_tiles);
    const int sp = t / (m_tiles * n_tiles);
    ti.group = sp;
    ti.kb_lo = sp * kb_per;
    ti.kb_n = min(kb_per, kb_main - ti.kb_lo);
    if (ti.kb_n < 0) ti.kb_n = 0;
    ti.extra = sp == 0;
    return ti;
  }
};

// acc (+ bias) (+ residual on the first res_cols columns) -> C as bf16 or fp32; optional SwiGLU
// output H for gate|up-interleaved columns (blocks of 16).
// swiglu_bwd: acc is d(silu(gate) * up) [M, N]; H holds the forward's gate|up pre-activations [M, 2N] (interleaved in
// blocks of 16) and C receives d(gate|up) [M, 2N] in the same layout, so the activation gradient never exists in
// memory as a separate tensor.
template <int BN, int CS = 2>
struct EpiStore {
  static constexpr int COL_SPLIT = CS;   // two epilogue warps per TMEM lane quarter, half of the columns each
  void* C;
  const __nv_bfloat16* R;
  __nv_bfloat16* H;
  const float* bias;
  int ldc, ldr, ldh;
  int M, N;
  int out_f32;
  int res_cols;
  int swiglu_bwd = 0;
  // Global operands of the NEXT 32-column chunk, loaded while the current chunk is converted and stored.
  // Residual (4 pieces): each thread reads its own row.  SwiGLU backward (8 pieces = 128 bytes of gate|up per row):
  // read cooperatively, 8 lanes per row, so that a warp-wide load touches 4 rows x 128 contiguous bytes instead of 32
  // rows x 16 bytes; the pieces reach their owning thread through a per-warp shared-memory slab, and the result leaves
  // the same way.  (One row per thread in global memory costs one L1 wavefront per lane and instruction; for this
  // epilogue, which moves 256 bytes per output row and chunk, that was more LSU time than the tile's main loop has.)
  // A second chunk of look-ahead was measured and does not help: these warps wait on issue latency, not on memory.
  uint4 pre[8];
  int pre_n = 0;     // pieces of `pre` that hold the chunk about to be processed (0: load at the point of use)

  __device__ __forceinline__ void issue(const TileInfo& ti, int row, int c) {
    const int gc = ti.n_blk * BN + c;
    pre_n = 0;
    if (c >= epi_col_end<BN, CS>() || gc + 32 > N) return;
    if (swiglu_bwd) {
      const int lane = row & 31;
      const int row0 = ti.m_blk * GEMM_BM + (row & ~31);       // first row of this warp's 32-row band
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int gr = row0 + i * 4 + (lane >> 3);
        pre[i] = gr < M ? *reinterpret_cast<const uint4*>(H + static_cast<size_t>(gr) * ldh + 2 * gc + (lane & 7) * 8)
                        : make_uint4(0, 0, 0, 0);
      }
      pre_n = 8;
      return;
    }
    const int gr = ti.m_blk * GEMM_BM + row;
    if (gr < M && R && gc + 32 <= res_cols) {
      const uint4* r = reinterpret_cast<const uint4*>(R + static_cast<size_t>(gr) * ldr + gc);
#pragma unroll
      for (int j = 0; j < 4; ++j) pre[j] = r[j];
      pre_n = 4;
    }
  }

  __device__ void tile_begin(const TileInfo& ti, int row) { issue(ti, row, epi_col_begin<BN, CS>()); }
  __device__ void tile_end(const TileInfo&, int) {}

  // d(gate|up) of one 32-column chunk of d(activation); executed by whole warps (rows past M are masked, not skipped)
  __device__ __forceinline__ void chunk_swiglu_bwd(const TileInfo& ti, int row, int c, uint32_t (&acc)[32]) {
    // per epilogue warp: 32 rows x 8 16-byte pieces; piece p of row r sits at r * 8 + (p ^ (r & 7)), which keeps both
    // access patterns (8 lanes along a row; 32 lanes down a column of pieces) free of bank conflicts without padding
    __shared__ uint4 s_slab[4 * CS][32 * 8];
    const int gc = ti.n_blk * BN + c;
    if (gc >= N) return;                     // warp-uniform
    const int lane = row & 31;
    uint4* sb = s_slab[epi_warp_slot()];
    const int row0 = ti.m_blk * GEMM_BM + (row & ~31);
    const int sw = lane & 7;
    // gate|up pieces -> slab, then every thread picks up its own row
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = i * 4 + (lane >> 3);
      sb[r * 8 + (sw ^ (r & 7))] = pre[i];
    }
    __syncwarp();
    issue(ti, row, c + 32);
    uint4 in[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) in[j] = sb[lane * 8 + (j ^ sw)];
    __syncwarp();
    // columns gc .. gc+31 of the activation map to columns 2gc .. 2gc+63 of gate|up: [g 0-15 | u 0-15 | g 16-31 | u 16-31]
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&in[blk * 4]);
      const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&in[blk * 4 + 2]);
      uint4 dg[2], du[2];
      uint32_t* dgp = reinterpret_cast<uint32_t*>(dg);
      uint32_t* dup = reinterpret_cast<uint32_t*>(du);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float2 g2 = __bfloat1622float2(gp[e]), u2 = __bfloat1622float2(up[e]);
        const float d0 = __uint_as_float(acc[blk * 16 + 2 * e]), d1 = __uint_as_float(acc[blk * 16 + 2 * e + 1]);
        // s = sigmoid(g); d gate = d u s (1 + g (1 - s)); d up = d g s   (approximate ex2 / rcp: the result is bf16)
        const float s0 = rcp_approx(1.f + __expf(-g2.x)), s1 = rcp_approx(1.f + __expf(-g2.y));
        const float a0 = d0 * s0, a1 = d1 * s1;
        const float t0 = fmaf(-g2.x, s0, g2.x), t1 = fmaf(-g2.y, s1, g2.y);
        const float p0 = a0 * u2.x, p1 = a1 * u2.y;
        dgp[e] = pack_bf16x2(fmaf(p0, t0, p0), fmaf(p1, t1, p1));
        dup[e] = pack_bf16x2(a0 * g2.x, a1 * g2.y);
      }
      sb[lane * 8 + ((blk * 4) ^ sw)] = dg[0];
      sb[lane * 8 + ((blk * 4 + 1) ^ sw)] = dg[1];
      sb[lane * 8 + ((blk * 4 + 2) ^ sw)] = du[0];
      sb[lane * 8 + ((blk * 4 + 3) ^ sw)] = du[1];
    }
    __syncwarp();
    __nv_bfloat16* dgu = reinterpret_cast<__nv_bfloat16*>(C) + 2 * gc + sw * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int r = i * 4 + (lane >> 3);
      if (row0 + r < M) *reinterpret_cast<uint4*>(dgu + static_cast<size_t>(row0 + r) * ldc) = sb[r * 8 + (sw ^ (r & 7))];
    }
    __syncwarp();
  }

  __device__ void chunk(const TileInfo& ti, int row, int c, uint32_t (&acc)[32]) {
    if (swiglu_bwd) {
      chunk_swiglu_bwd(ti, row, c, acc);
      return;
    }
    const int gr = ti.m_blk * GEMM_BM + row;
    const int gc = ti.n_blk * BN + c;
    if (gr >= M || gc >= N) return;
    const bool full = (gc + 32 <= N);
    uint4 cur[4];
    const int cur_n = pre_n;
#pragma unroll
    for (int j = 0; j < 4; ++j) cur[j] = pre[j];
    issue(ti, row, c + 32);
    if (bias) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (full || gc + j < N) acc[j] = __float_as_uint(__uint_as_float(acc[j]) + __ldg(bias + gc + j));
    }
    if (R && gc < res_cols) {
      const __nv_bfloat16* r = R + static_cast<size_t>(gr) * ldr + gc;
      if (gc + 32 <= res_cols) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 rv = cur_n == 4 ? cur[j >> 3] : *reinterpret_cast<const uint4*>(r + j);
          const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(rp[e]);
            acc[j + 2 * e] = __float_as_uint(__uint_as_float(acc[j + 2 * e]) + f.x);
            acc[j + 2 * e + 1] = __float_as_uint(__uint_as_float(acc[j + 2 * e + 1]) + f.y);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gc + j < res_cols) acc[j] = __float_as_uint(__uint_as_float(acc[j]) + __bfloat162float(r[j]));
      }
    }
    if (out_f32) {
      float* out = reinterpret_cast<float*>(C) + static_cast<size_t>(gr) * ldc + gc;
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<uint4*>(out + j) = make_uint4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gc + j < N) out[j] = __uint_as_float(acc[j]);
      }
      return;
    }
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(C) + static_cast<size_t>(gr) * ldc + gc;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1]));
        v.y = pack_bf16x2(__uint_as_float(acc[j + 2]), __uint_as_float(acc[j + 3]));
        v.z = pack_bf16x2(__uint_as_float(acc[j + 4]), __uint_as_float(acc[j + 5]));
        v.w = pack_bf16x2(__uint_as_float(acc[j + 6]), __uint_as_float(acc[j + 7]));
        *reinterpret_cast<uint4*>(out + j) = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (gc + j < N) out[j] = __float2bfloat16(__uint_as_float(acc[j]));
    }
    if (H && full) {
      // slab = [gate 0..15 | up 0..15]; the activation uses the bf16-rounded values so that a
      // backward pass that re-reads GU sees exactly what produced H.
      __nv_bfloat16* h = H + static_cast<size_t>(gr) * ldh + (gc >> 1);
      uint32_t hv[8];
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        float g0 = __bfloat162float(__float2bfloat16(__uint_as_float(acc[j])));
        float g1 = __bfloat162float(__float2bfloat16(__uint_as_float(acc[j + 1])));
        float u0 = __bfloat162float(__float2bfloat16(__uint_as_float(acc[16 + j])));
        float u1 = __bfloat162float(__float2bfloat16(__uint_as_float(acc[16 + j + 1])));
        float h0 = g0 * rcp_approx(1.f + __expf(-g0)) * u0;
        float h1 = g1 * rcp_approx(1.f + __expf(-g1)) * u1;
        hv[j >> 1] = pack_bf16x2(h0, h1);
      }
      *reinterpret_cast<uint4*>(h) = make_uint4(hv[0], hv[1], hv[2], hv[3]);
      *reinterpret_cast<uint4*>(h + 8) = make_uint4(hv[4], hv[5], hv[6], hv[7]);
    }
  }
};

// Grouped (per-expert) GEMM: rows are sorted by expert and every expert's segment is padded to a
// multiple of 128 rows, so an M tile belongs to exactly one expert, read from tile_expert[m_blk]
// (-1: tile beyond the last segment, nothing to do).  B and B2 hold the experts' matrices stacked
// along rows.
struct SchedGrouped {
  const int* tile_expert;
  int m_tiles, n_tiles, b_rows_per_expert;
  __device__ int tiles_for_cta(int cta, int ncta) const {
    const int total = m_tiles * n_tiles;
    return cta < total ? (total - cta + ncta - 1) / ncta : 0;
  }
  __device__ TileInfo get(int cta, int ncta, int i) const {
    const int t = cta + i * ncta;
    TileInfo ti = make_tile(t % m_tiles, t / m_tiles);
    const int e = __ldg(tile_expert + ti.m_blk);
    ti.group = e;
    if (e < 0) {
      ti.kb_n = 0;
      ti.extra = 0;
    } else {
      ti.b_row = e * b_rows_per_expert;
    }
    return ti;
  }
};

template <int BN>
struct EpiGrouped {
  EpiStore<BN, 1> st;
  __device__ void tile_begin(const TileInfo& ti, int row) {
    if (ti.group >= 0) st.tile_begin(ti, row);
  }
  __device__ void tile_end(const TileInfo&, int) {}
  __device__ void chunk(const TileInfo& ti, int row, int c, uint32_t (&acc)[32]) {
    if (ti.group >= 0) st.chunk(ti, row, c, acc);
  }
};

// Split-K partial: fp32 atomic accumulation into a zero-initialised workspace [M, ldw].
template <int BN>
struct EpiAtomic {
  float* W;
  int ldw, M, N;
  __device__ void tile_begin(const TileInfo&, int) {}
  __device__ void tile_end(const TileInfo&, int) {}
  __device__ void chunk(const TileInfo& ti, int row, int c, uint32_t (&acc)[32]) {
    const int gr = ti.m_blk * GEMM_BM + row;
    const int gc = ti.n_blk * BN + c;
    if (gr >= M || gc >= N || ti.kb_n == 0) return;
    float* w = W + static_cast<size_t>(gr) * ldw + gc;
    if (gc + 32 <= N) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        atomicAdd(reinterpret_cast<float4*>(w + j),
                  make_float4(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1]), __uint_as_float(acc[j + 2]),
                              __uint_as_float(acc[j + 3])));
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (gc + j < N) atomicAdd(w + j, __uint_as_float(acc[j]));
    }
  }
};

}  // namespace artb
