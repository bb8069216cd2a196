// Device-side index checks that are compiled in with -DARTB_BOUNDS_CHECK (python -m art_b200.build --checked builds the
// whole kernel library that way as libartb_kernels_checked.so; ARTB_BOUNDS_CHECK=1 in the environment loads it).
//
// Every index that a kernel takes from memory (cache slot, block-table entry, row index, adapter slot) goes through
// index_ok(): in a checked build a value outside [0, n) records ST_BOUNDS in the status word the host polls after a
// step and the access is skipped; nothing traps and the context stays usable.  In the normal build the function is
// the constant `true` and costs nothing.  This is the stand-in for a memory checker on hardware where none can be run
// over the kernels.  The reference has no native code to check (pure Python; its concurrency rests on one asyncio
// loop per process, src/art/local/state.py:28).
#pragma once
#include "ptx_sm100.cuh"

namespace artb {

#ifdef ARTB_BOUNDS_CHECK
constexpr bool BOUNDS_CHECKED = true;
#else
constexpr bool BOUNDS_CHECKED = false;
#endif

__device__ __forceinline__ bool index_ok(long long i, long long n, int* status) {
  if (BOUNDS_CHECKED && (i < 0 || i >= n)) {
    if (status) atomicMax(status, ST_BOUNDS);
    return false;
  }
  return true;
}

}  // namespace artb
