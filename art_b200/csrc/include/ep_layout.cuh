// Expert-parallel all-to-all: shared layout of the symmetric region and of the per-call plan.
//
// P ranks, E experts, E_l = E / P experts per rank (expert e lives on rank e / E_l).  Every rank
// routes its own tokens, sorts them by expert (segments padded to 128 rows, as on one GPU) and
// then
//   dispatch: pushes the rows of expert e into the owner's receive staging buffer, behind the
//             rows the lower-numbered ranks send for e;
//   return:   the owner pushes the expert outputs back to the row each came from.
// All ranks first all-gather their per-expert counts (P x E int32 through the symmetric buffer),
// from which every rank derives every offset it needs without further communication.
//
// Symmetric region (same byte offsets on every rank; `par` = call parity for double buffering):
//   cnt      int32  [2][P][E]        counts written by each source
//   cnt_flag uint32 [P]              epoch of the last counts written by each source
//   recv     bf16   [2][cap_recv][D] dispatch staging at the expert owner
//   dflag    uint32 [E_l][P]         dispatch arrival: epoch per (local expert, source)
//   ddone    uint32 [P]              "my recv staging of call e is consumed", published to all
//   ret      bf16   [2][cap_src][D]  return staging at the token owner
//   rflag    uint32 [P]              return arrival: epoch per expert rank
//   rdone    uint32 [P]
#pragma once
#include "symm.cuh"

namespace artb {

constexpr int EP_MAX_RANKS = 8;
constexpr int EP_MAX_EXPERTS = 256;

struct EpPeers {
  char* base[EP_MAX_RANKS];
};

__device__ __forceinline__ char* ep_base(const EpPeers& pt, int i) {
  char* b = pt.base[0];
#pragma unroll
  for (int p = 1; p < EP_MAX_RANKS; ++p)
    if (p == i) b = pt.base[p];
  return b;
}

// Per-call plan, all device int32 arrays owned by the caller (private memory):
struct EpPlan {
  int* cnt_all;        // [P][E]      counts of every source
  int* send_off;       // [E]         row in the owner's recv staging where MY rows of expert e start
  int* seg_off;        // [E_l + 1]   padded segment offsets of my local experts in recv order
  int* tile_expert;    // [cap_tiles] local expert of each 128-row tile of recv (-1 beyond the end)
  int* src_start;      // [E_l][P]    offset inside local expert j's segment where source s starts
  int* src_seg_off;    // [P][E_l]    row in SOURCE s's sorted order where its segment of my expert j starts
  int* real_rows;      // [E_l]       rows actually received for local expert j (sum over sources)
};

}  // namespace artb
