// Shared declarations of the symmetric-memory layer: the per-rank state behind the opaque handle
// of the host API, the table of peer base pointers that kernels receive, and the system-scope
// release/acquire accessors used for flags that another GPU writes or reads.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace artb {

constexpr int MAX_RANKS = 16;
constexpr int PAD_SLOTS = 64;   // uint64 epoch slots per rank (slot q of channel c at c*16+q)

struct PeerTable {
  void* base[MAX_RANKS];      // data area of every rank (own included)
  uint64_t* pad[MAX_RANKS];   // signal pad of every rank
};

__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Deadline of a bounded wait of `budget_us` microseconds, and its check (polled every 64th iteration; an iteration cap
// stands behind it, so the wait ends even where the timer does not advance).
struct WaitBudget {
  uint64_t t0, budget_ns;
  uint32_t it = 0;
  __device__ __forceinline__ explicit WaitBudget(uint32_t budget_us)
      : t0(global_timer_ns()), budget_ns(static_cast<uint64_t>(budget_us) * 1000ull) {}
  __device__ __forceinline__ bool expired() {
    ++it;
    if (it > 0xF0000000u) return true;
    return (it & 63u) == 0 && global_timer_ns() - t0 > budget_ns;
  }
};

// Bounded wait until *p >= target: gives up after `budget_us` microseconds of wall time (callers pass wait_ms * 1000).
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* p, uint32_t target, uint32_t budget_us) {
  if (static_cast<int32_t>(ld_acquire_sys_u32(p) - target) >= 0) return true;
  WaitBudget w(budget_us);
  while (static_cast<int32_t>(ld_acquire_sys_u32(p) - target) < 0) {
    if (w.expired()) return false;
    __nanosleep(64);
  }
  return true;
}

struct SymmState {
  int rank = -1, world = 0;
  size_t data_bytes = 0;
  void* local = nullptr;          // cudaMalloc'd: data area + pad
  PeerTable table;
  void* opened[MAX_RANKS];
  uint32_t* gate = nullptr;
  uint64_t epoch = 0;
};

}  // namespace artb
