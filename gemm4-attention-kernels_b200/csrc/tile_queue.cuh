// Dynamic tile scheduling for persistent CTA pairs.
//
// One thread of the leader CTA draws tile indices from a global counter and publishes them to both CTAs
// of the pair through a two-entry queue in shared memory; every role (TMA producer, MMA issuer, epilogue
// warps) of both CTAs reads each entry once. The first tile of a pair is its own index, so no atomic sits
// in front of the first load; later tiles come from `n_pairs + atomicAdd(counter, 1)`. A pair that ends
// early simply draws more tiles, which is what balances tiles of unequal weight (causal masks, packed
// sequences of different lengths). The counter must be zero when the kernel starts; the last pair to draw from
// it puts it back to zero (counted in a second word), so the next launch on the same workspace needs no memset.
//
// Every wait is bounded (mbar_wait): a role that gives up sets the CTA's abort flag and returns -1.
#pragma once
#include "ptx.cuh"

namespace sd {

struct TileQueue {
  uint32_t idx;           // shared address of int[2] (this CTA)
  uint32_t full;          // shared address of 2 mbarriers (this CTA), count 1
  uint32_t empty_leader;  // cluster address of 2 mbarriers in the leader CTA, count = consumers of both CTAs
};
constexpr int kTileQueueBytes = 8 + 16 + 16;  // idx[2], full[2], empty[2]

__device__ __forceinline__ TileQueue tq_make(uint32_t base) {
  TileQueue q;
  q.idx = base;
  q.full = base + 8;
  q.empty_leader = mapa_u32(base + 24, 0);
  return q;
}
// one thread per CTA, before the cluster-wide sync that publishes the barriers
__device__ __forceinline__ void tq_init(uint32_t base, int consumers_in_pair) {
  mbar_init(base + 8, 1);
  mbar_init(base + 16, 1);
  mbar_init(base + 24, consumers_in_pair);
  mbar_init(base + 32, consumers_in_pair);
}

// Scheduler loop, run by ONE thread of the leader CTA. Ends after publishing the first index >= total.
__device__ __forceinline__ void tq_schedule(uint32_t base, int* counter, int* done, int pair_id, int n_pairs,
                                            int total, volatile int* abort_flag, int* status) {
  const uint32_t peer_idx = mapa_u32(base, 1), peer_full = mapa_u32(base + 8, 1);
  for (int n = 0;; ++n) {
    const uint32_t slot = n & 1, ph = (n >> 1) & 1;
    if (!mbar_wait<true>(base + 24 + 8 * slot, ph ^ 1u, abort_flag, status, ST_TIMEOUT_PEER)) return;
    const int idx = n == 0 ? pair_id : n_pairs + atomicAdd(counter, 1);
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(base + 4 * slot), "r"(idx) : "memory");
    st_cluster_u32(peer_idx + 4 * slot, static_cast<uint32_t>(idx));
    mbar_arrive_cluster(mapa_u32(base + 8 + 8 * slot, 0));  // release at cluster scope orders the stores above
    mbar_arrive_cluster(peer_full + 8 * slot);
    if (idx >= total) {
      // every pair ends with exactly one draw >= total; after the last of them nobody touches the counter again
      __threadfence();
      if (atomicAdd(done, 1) == n_pairs - 1) {
        *counter = 0;
        *done = 0;
        __threadfence();
      }
      return;
    }
  }
}

// n-th tile index of this pair, or -1 after a failed wait. Call with `whole_warp` = true from all 32 lanes
// of a warp role (one arrival per warp), or false from a single-thread role.
__device__ __forceinline__ int tq_fetch(const TileQueue& q, int n, bool whole_warp, volatile int* abort_flag,
                                        int* status) {
  const uint32_t slot = n & 1, ph = (n >> 1) & 1;
  bool ok = mbar_wait<true>(q.full + 8 * slot, ph, abort_flag, status, ST_TIMEOUT_PEER);
  if (whole_warp) ok = __all_sync(0xffffffffu, ok);
  if (!ok) return -1;
  int idx;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(idx) : "r"(q.idx + 4 * slot) : "memory");
  if (whole_warp) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive_cluster(q.empty_leader + 8 * slot);
  } else {
    mbar_arrive_cluster(q.empty_leader + 8 * slot);
  }
  return idx;
}

}  // namespace sd
