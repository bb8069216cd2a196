// Schedule / communication / epilogue policies that turn the tcgen05 GEMM pipeline into the two
// tensor-parallel fused kernels:
//
//   all-gather -> GEMM   (column-parallel linear, activations sharded along tokens)
//   GEMM -> reduce-scatter (row-parallel linear, output sharded along tokens)
//
// All cross-GPU traffic is plain st/ld through peer pointers of a symmetric buffer; the TMA
// loads of the GEMM only ever read this GPU's own memory (remote shards are pushed into the local
// copy of the gathered matrix first).  Flags carry a monotonically increasing call number
// ("epoch"), so nothing is reset between calls; buffers are double-buffered by epoch parity and a
// per-rank "done" word tells writers that the call two epochs back has been fully consumed.
// Every wait is bounded and reports ST_TIMEOUT_PEER.
#pragma once
#include "gemm_epilogue.cuh"
#include "symm.cuh"

namespace artb {

constexpr int TP_MAX = 8;
constexpr int TP_PUSH_ROWS = 32;   // rows per push unit / arrival flag

// Token segments (one per rank) are visited in rotated order; inside a segment the tiles follow the grouped order
// of raster_tile (bands of group_m tile rows, M fastest inside a band), so that the band of A in use stays in L2.
// first_off = 0: own segment first (all-gather: local data is there already);
// first_off = 1: own segment last  (reduce-scatter: peers' partials arrive while we compute theirs).
struct SchedSegRot {
  int seg_m_tiles, n_tiles, world, rank, first_off, group_m;
  // Reduce-scatter only (first_off = 1): instead of all peers' tiles first and the own segment last, the own tiles are
  // woven in `lag` tile positions behind the peers' tiles of the same position, so that the partial sums cross
  // NVLink during the whole kernel rather than during its first (world-1)/world, which for short reductions is more
  // than the link carries in that time.  The peers run the mirror-image order, so the partial an own tile adds was
  // pushed lag * world tiles (a few grid waves) earlier.  0 or >= tiles per segment: peers first, own last.
  int lag = 0;
  __device__ int tiles_for_cta(int cta, int ncta) const {
    const int total = seg_m_tiles * n_tiles * world;
    return cta < total ? (total - cta + ncta - 1) / ncta : 0;
  }
  __device__ TileInfo get(int cta, int ncta, int i) const {
    const int t = cta + i * ncta;
    const int per_seg = seg_m_tiles * n_tiles;
    int seg, pos;
    if (lag <= 0 || lag >= per_seg || first_off != 1 || world < 2) {
      const int si = t / per_seg;
      pos = t - si * per_seg;
      seg = (rank + first_off + si) % world;
    } else {
      const int others = world - 1;
      const int a_end = lag * others;                  // positions [0, lag): peers' tiles only
      if (t < a_end) {
        pos = t / others;
        seg = (rank + 1 + t % others) % world;
      } else {
        const int u = t - a_end, b_len = (per_seg - lag) * world;
        if (u < b_len) {                               // positions [lag, per_seg): peers' tiles + the own tile `lag` behind
          const int k = u % world;
          pos = lag + u / world;
          if (k < others) {
            seg = (rank + 1 + k) % world;
          } else {
            seg = rank;
            pos -= lag;
          }
        } else {                                       // the last `lag` own tiles
          seg = rank;
          pos = per_seg - lag + (u - b_len);
        }
      }
    }
    int m, n;
    raster_tile(pos, seg_m_tiles, n_tiles, group_m, m, n);
    TileInfo ti = make_tile(seg * seg_m_tiles + m, n);
    ti.group = seg;
    return ti;
  }
};

struct TpPeers {
  char* base[TP_MAX];   // data area of every rank's symmetric buffer
};

// Select chain instead of a dynamic index, so that a policy object holding the table can stay in
// registers.
__device__ __forceinline__ char* tp_base(const TpPeers& pt, int i) {
  char* b = pt.base[0];
#pragma unroll
  for (int p = 1; p < TP_MAX; ++p)
    if (p == i) b = pt.base[p];
  return b;
}

// Publishes "this rank has finished call `epoch`" to every peer once the last CTA retires.
__device__ __forceinline__ void tp_publish_done(const TpPeers& pt, long off_done, int rank, int world,
                                                uint32_t epoch, unsigned int* cta_counter) {
  __threadfence();
  const unsigned int prev = atomicAdd(cta_counter, 1u);
  if (prev + 1 == gridDim.x) {
    *cta_counter = 0;   // the next launch on this stream starts after this one has ended
    __threadfence_system();
    for (int p = 0; p < world; ++p)
      st_release_sys_u32(reinterpret_cast<uint32_t*>(pt.base[p] + off_done) + rank, epoch);
  }
}

// ------------------------------------------------------------------------------ all-gather side
// Symmetric layout (same offsets on every rank): X [world * m_seg, K] bf16 dense at off_x,
// optional T [world * m_seg, kt] bf16 dense at off_t (the low-rank LoRA activations, gathered with
// X), arrival flags uint32 [world][m_seg / 32] at off_flag, done words uint32 [world] at off_done.
// The caller has written its own shard into rows [rank * m_seg, (rank+1) * m_seg) of the local X / T.
struct AgComm {
  static constexpr int THREADS = 64;   // two warps; eight 16-byte loads in flight per thread
  TpPeers pt;
  long off_x, off_t, off_flag, off_done;
  int rank, world, m_seg;
  int row_bytes_x, row_bytes_t;   // dense row sizes (multiples of 16); row_bytes_t == 0: no T
  uint32_t epoch, spin;
  unsigned int* cta_counter;

  __device__ void copy_rows(char* dst, const char* src, long bytes, int tid) const {
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    const long n = bytes >> 4;
    long i = tid;
    for (; i + 7 * THREADS < n; i += 8 * THREADS) {
      uint4 v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = s[i + j * THREADS];
#pragma unroll
      for (int j = 0; j < 8; ++j) d[i + j * THREADS] = v[j];
    }
    for (; i < n; i += THREADS) d[i] = s[i];
  }

  __device__ void push(int tid, int* status) const {
    if (world == 1) return;
    const int units = m_seg / TP_PUSH_ROWS;
    __shared__ int s_ok;
    // peers must have consumed the call that last used this parity of the buffer
    if (tid == 0) {
      int ok = 1;
      const uint32_t* done = reinterpret_cast<const uint32_t*>(pt.base[rank] + off_done);
      if (epoch > 2)
        for (int p = 0; p < world; ++p)
          if (p != rank && !wait_flag_ge(done + p, epoch - 2, spin)) ok = 0;
      if (!ok) atomicMax(status, ST_TIMEOUT_PEER);
      s_ok = ok;
    }
    asm volatile("bar.sync 1, 64;" ::: "memory");
    if (!s_ok) return;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      const long row0 = static_cast<long>(rank) * m_seg + static_cast<long>(u) * TP_PUSH_ROWS;
      for (int i = 1; i < world; ++i) {
        const int p = (rank - i + world) % world;   // rank-1 consumes our segment first
        copy_rows(pt.base[p] + off_x + row0 * row_bytes_x, pt.base[rank] + off_x + row0 * row_bytes_x,
                  static_cast<long>(TP_PUSH_ROWS) * row_bytes_x, tid);
        if (row_bytes_t)
          copy_rows(pt.base[p] + off_t + row0 * row_bytes_t, pt.base[rank] + off_t + row0 * row_bytes_t,
                    static_cast<long>(TP_PUSH_ROWS) * row_bytes_t, tid);
        __threadfence_system();
        asm volatile("bar.sync 1, 64;" ::: "memory");
        if (tid == 0)
          st_release_sys_u32(reinterpret_cast<uint32_t*>(pt.base[p] + off_flag) + rank * units + u, epoch);
      }
    }
  }

  // producer lane, before the first load of a tile
  __device__ bool ready(const TileInfo& ti) const {
    const int seg = ti.group;
    if (seg == rank) return true;
    const int units = m_seg / TP_PUSH_ROWS;
    const int u0 = (ti.m_blk * GEMM_BM - seg * m_seg) / TP_PUSH_ROWS;
    const uint32_t* fl = reinterpret_cast<const uint32_t*>(pt.base[rank] + off_flag) + seg * units + u0;
    for (int j = 0; j < GEMM_BM / TP_PUSH_ROWS; ++j)
      if (!wait_flag_ge(fl + j, epoch, spin)) return false;
    fence_proxy_async_all();   // peer's generic-proxy stores -> this CTA's TMA (async proxy) reads
    return true;
  }

  __device__ void finish(int* /*status*/) const { tp_publish_done(pt, off_done, rank, world, epoch, cta_counter); }
};

// -------------------------------------------------------------------------- reduce-scatter side
// Symmetric layout: staging bf16 [world-1][m_seg][N] at off_stage (slot s of owner o holds the
// partial of rank (o + 1 + s) % world), flags uint32 [world-1][tile_cap][8] at off_flag (one per epilogue warp), done
// words at off_done.  Output: out[m_seg, N] bf16 = sum over ranks (+ residual shard R).
struct RsComm {
  static constexpr int THREADS = 0;
  TpPeers pt;
  long off_done;
  int rank, world;
  uint32_t epoch;
  unsigned int* cta_counter;
  __device__ void push(int, int*) const {}
  __device__ bool ready(const TileInfo&) const { return true; }
  __device__ void finish(int*) const { tp_publish_done(pt, off_done, rank, world, epoch, cta_counter); }
};

template <int BN>
struct EpiReduceScatter {
  static constexpr int COL_SPLIT = 2;   // two epilogue warps per TMEM lane quarter, half of the columns each
  // remote tiles leave through a shared-memory slab that is flushed after every SECOND 32-column chunk
  static_assert(BN % 128 == 0, "EpiReduceScatter needs an even number of 32-column chunks per epilogue warp");
  TpPeers pt;
  long off_stage, off_flag, off_done;
  __nv_bfloat16* out;
  const __nv_bfloat16* R;
  int ldc, ldr, N, m_seg, n_tiles, tile_cap, rank, world;
  uint32_t epoch, spin;
  int* status;
  // per-tile state
  int own, lrow;
  __nv_bfloat16* stage;   // first row of this warp's 32-row band: in the owner's staging slot (remote tile)
                          // or in slot 0 of the local staging (own tile)
  uint32_t* flag;         // remote: flag to publish; own: flag of slot 0 to wait on
  // Own tiles: the staged partial of slot 0 and the residual of the NEXT 32-column chunk, loaded while the current
  // chunk is summed and stored.  A thread reads its own row, so issued at the point of use these loads cost one DRAM
  // round trip per chunk, which for short reductions (K of a few thousand) is longer than the tile's main loop.
  uint4 pre[8];
  int pre_ok = 0;
  uint32_t done_seen = 0;   // bit seg: the owner's "done" word was already checked in this launch

  // Cooperative form: the warp's 32 rows x 64 bytes of the staged partial, and the same of the residual, are read
  // with four lanes per row (a warp-wide load touches 8 rows x 64 contiguous bytes instead of 32 rows x 16 bytes);
  // lane holds row i * 8 + lane / 4, 16-byte piece lane % 4, for i = 0..3.  One row per lane costs an L1 wavefront per
  // lane and instruction, and this epilogue has twelve such instructions per chunk: measured on one rank, the tensor
  // pipe of the reduce-scatter kernel was busy 59 % of the time against 81 % for the plain-store kernels.
  __device__ __forceinline__ void issue(const TileInfo& ti, int row, int c) {
    const int gc = ti.n_blk * BN + c;
    pre_ok = 0;
    if (!own || c >= epi_col_end<BN, COL_SPLIT>() || gc + 32 > N) return;
    const int lane = row & 31;
    const int p8 = (lane & 3) * 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i * 8 + (lane >> 2);
      pre[i] = world > 1 ? __ldcg(reinterpret_cast<const uint4*>(stage + static_cast<size_t>(r) * N + gc + p8))
                         : make_uint4(0, 0, 0, 0);
      pre[4 + i] = R ? *reinterpret_cast<const uint4*>(R + static_cast<size_t>(lrow - lane + r) * ldr + gc + p8)
                     : make_uint4(0, 0, 0, 0);
    }
    pre_ok = 1;
  }

  __device__ void tile_begin(const TileInfo& ti, int row) {
    const int seg = ti.group;
    const int q = (row >> 5) & 3, lane = row & 31;
    const int ws = epi_warp_slot();     // the owner's warp of the same slot reads what this warp stages
    own = seg == rank;
    const int lrow0 = ti.m_blk * GEMM_BM - seg * m_seg;
    lrow = lrow0 + row;
    const int tile_local = (lrow0 / GEMM_BM) * n_tiles + ti.n_blk;
    int ok = 1;
    if (!own) {
      const int slot = (rank - seg - 1 + world) % world;
      stage = reinterpret_cast<__nv_bfloat16*>(tp_base(pt, seg) + off_stage) +
              (static_cast<size_t>(slot) * m_seg + lrow0 + q * 32) * N;
      flag = reinterpret_cast<uint32_t*>(tp_base(pt, seg) + off_flag) +
             (static_cast<size_t>(slot) * tile_cap + tile_local) * 8 + ws;
      // the owner must have consumed the call that last used this parity of its staging buffer (checked once per
      // launch and owner: the word only grows)
      if (epoch > 2 && !((done_seen >> seg) & 1u)) {
        if (lane == 0)
          ok = wait_flag_ge(reinterpret_cast<const uint32_t*>(tp_base(pt, rank) + off_done) + seg, epoch - 2, spin);
        done_seen |= 1u << seg;
      }
    } else {
      stage = reinterpret_cast<__nv_bfloat16*>(tp_base(pt, rank) + off_stage) +
              static_cast<size_t>(lrow0 + q * 32) * N;
      flag = reinterpret_cast<uint32_t*>(tp_base(pt, rank) + off_flag) + static_cast<size_t>(tile_local) * 8 + ws;
      if (lane == 0)
        for (int s = 0; s < world - 1; ++s)
          if (!wait_flag_ge(flag + static_cast<size_t>(s) * tile_cap * 8, epoch, spin)) ok = 0;
    }
    if (lane == 0 && !ok) atomicMax(status, ST_TIMEOUT_PEER);
    __syncwarp();
    issue(ti, row, epi_col_begin<BN, COL_SPLIT>());       // after the flags: the staged partials are complete
  }

  __device__ void chunk(const TileInfo& ti, int row, int c, uint32_t (&acc)[32]) {
    // per warp: 32 rows x 8 16-byte pieces; piece p of row r at r * 8 + (p ^ (r & 7)) (no padding)
    __shared__ uint4 s_buf[8][32 * 8];
    uint4* sb = s_buf[epi_warp_slot()];
    const int gc = ti.n_blk * BN + c;
    const int lane = row & 31, sw = lane & 7;
    if (!own) {
      // Remote tile: the partial goes to the owner as bf16.  A thread holds one row, so a direct
      // store would scatter 16-byte pieces over 32 rows; instead two 32-column slabs are parked in
      // shared memory and written out with 8 lanes covering 128 contiguous bytes of a row.
      const int half = (c >> 5) & 1;
      if (gc < N) {
        uint4* w = sb + lane * 8;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(acc[8 * j]), __uint_as_float(acc[8 * j + 1]));
          v.y = pack_bf16x2(__uint_as_float(acc[8 * j + 2]), __uint_as_float(acc[8 * j + 3]));
          v.z = pack_bf16x2(__uint_as_float(acc[8 * j + 4]), __uint_as_float(acc[8 * j + 5]));
          v.w = pack_bf16x2(__uint_as_float(acc[8 * j + 6]), __uint_as_float(acc[8 * j + 7]));
          w[(half * 4 + j) ^ sw] = v;
        }
      }
      if (half == 1) {
        __syncwarp();
        const int gc0 = gc - 32;
        int pieces = (N - gc0) >> 3;   // N is a multiple of 8
        pieces = pieces > 8 ? 8 : pieces;
        const int j = lane & 7;
        if (j < pieces) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + (lane >> 3);
            const uint4 v = sb[r * 8 + (j ^ (r & 7))];
            *reinterpret_cast<uint4*>(stage + static_cast<size_t>(r) * N + gc0 + j * 8) = v;
          }
        }
        __syncwarp();
      }
      return;
    }
    if (gc >= N) return;          // warp-uniform
    auto add8 = [&](const uint4& rv, int j) {
      const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(rp[e]);
        acc[j + 2 * e] = __float_as_uint(__uint_as_float(acc[j + 2 * e]) + f.x);
        acc[j + 2 * e + 1] = __float_as_uint(__uint_as_float(acc[j + 2 * e + 1]) + f.y);
      }
    };
    const __nv_bfloat16* mine = stage + static_cast<size_t>(lane) * N + gc;
    if (pre_ok) {
      // Full chunk, operands prefetched cooperatively: pieces -> slab (staged in 0..3, residual in 4..7 of a row),
      // every thread picks up its own row, and the result leaves through the slab the same way.
      const int p = lane & 3;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i * 8 + (lane >> 2);
        sb[r * 8 + (p ^ (r & 7))] = pre[i];
        sb[r * 8 + ((4 + p) ^ (r & 7))] = pre[4 + i];
      }
      __syncwarp();
      issue(ti, row, c + 32);
      uint4 in[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) in[j] = sb[lane * 8 + (j ^ sw)];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        add8(in[j], 8 * j);          // zeros when world == 1
        add8(in[4 + j], 8 * j);      // zeros without a residual
      }
      for (int s = 1; s < world - 1; ++s) {       // further peers' partials: one row per lane
        const __nv_bfloat16* q = mine + static_cast<size_t>(s) * m_seg * N;
#pragma unroll
        for (int j = 0; j < 4; ++j) add8(__ldcg(reinterpret_cast<const uint4*>(q + 8 * j)), 8 * j);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(acc[8 * j]), __uint_as_float(acc[8 * j + 1]));
        v.y = pack_bf16x2(__uint_as_float(acc[8 * j + 2]), __uint_as_float(acc[8 * j + 3]));
        v.z = pack_bf16x2(__uint_as_float(acc[8 * j + 4]), __uint_as_float(acc[8 * j + 5]));
        v.w = pack_bf16x2(__uint_as_float(acc[8 * j + 6]), __uint_as_float(acc[8 * j + 7]));
        sb[lane * 8 + (j ^ sw)] = v;     // own row: no other thread reads these pieces before the barrier below
      }
      __syncwarp();
      __nv_bfloat16* o = out + static_cast<size_t>(lrow - lane) * ldc + gc + p * 8;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = i * 8 + (lane >> 2);
        *reinterpret_cast<uint4*>(o + static_cast<size_t>(r) * ldc) = sb[r * 8 + (p ^ (r & 7))];
      }
      __syncwarp();
      return;
    }
    // ragged chunk at the right edge of the matrix: one row per lane, loads at the point of use
    for (int s = 0; s < world - 1; ++s) {
      const __nv_bfloat16* q = mine + static_cast<size_t>(s) * m_seg * N;
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        if (gc + j < N) add8(__ldcg(reinterpret_cast<const uint4*>(q + j)), j);
    }
    if (R) {
      const __nv_bfloat16* r = R + static_cast<size_t>(lrow) * ldr + gc;
#pragma unroll
      for (int j = 0; j < 32; j += 8)
        if (gc + j < N) add8(*reinterpret_cast<const uint4*>(r + j), j);
    }
    __nv_bfloat16* o = out + static_cast<size_t>(lrow) * ldc + gc;
#pragma unroll
    for (int j = 0; j < 32; j += 8)
      if (gc + j < N) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1]));
        v.y = pack_bf16x2(__uint_as_float(acc[j + 2]), __uint_as_float(acc[j + 3]));
        v.z = pack_bf16x2(__uint_as_float(acc[j + 4]), __uint_as_float(acc[j + 5]));
        v.w = pack_bf16x2(__uint_as_float(acc[j + 6]), __uint_as_float(acc[j + 7]));
        *reinterpret_cast<uint4*>(o + j) = v;
      }
  }

  __device__ void tile_end(const TileInfo&, int row) {
    if (own) return;
    // a tile's flag is published at once (a system-scope fence, one NVLink round trip): holding it back to share the
    // fence between several tiles was measured and is slower, because the owner then waits for it
    __threadfence_system();
    __syncwarp();
    if ((row & 31) == 0) st_release_sys_u32(flag, epoch);
  }
};

}  // namespace artb
