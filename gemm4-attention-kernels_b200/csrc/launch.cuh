// Host-side launchers shared between the C-ABI file and the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>

#include <atomic>

#include "../../include/splitd_attn.h"
#include "common.cuh"

namespace sd {

int fail(int code, const char* fmt, ...);
int make_tmap(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const int64_t* strides_elems,
              const uint32_t* box, const char* what);
// rows_per_cta: packed query rows one CTA of a pair owns (64 or 128); heads fold when the group divides 64
void fill_geom(const splitd_params* p, TileGeom& g, int rows_per_cta = kRowsPerCta);
int make_q_tmap(CUtensorMap* map, const void* base, const splitd_params* p, const TileGeom& g, const int64_t* st,
                int box_pos, const char* what);
int make_kv_tmap(CUtensorMap* map, const void* base, const splitd_params* p, const int64_t* st, int box_rows,
                 const char* what);

// How the backward cuts its (head unit) x (row tile) space into chunks whose P / dS planes fit the workspace.
struct BwdPlan {
  size_t head_bytes;   // work counters + per-group maxima
  size_t copy_q_bytes, copy_k_bytes;  // fp16 copies: dO and Q (each copy_q_bytes), K
  size_t fixed_bytes;  // head + the three copies: everything in front of the accumulators and the planes
  size_t carry_bytes;  // fp32 dK / dV accumulators between chunks (used by mode 3 only)
  size_t tile_bytes;   // both planes of one 128-row tile
  size_t full_bytes;   // planes of the whole problem
  int64_t g_end;       // row tiles per head unit (packed layout: upper bound over all sequences)
  int64_t pitch;       // elements per plane row
  int head_units, upk; // upk: head units per KV head (1 when the query heads fold into the rows)
  int row_tiles_seq;   // batched layout: row tiles per sequence; 0 = packed
  int batch;
  int mode;            // 0 one chunk; 1 whole KV heads; 2 one KV head x some batches; 3 one head unit x a row range
  int n_chunks, kv_per_chunk, batches_per_chunk, slices, use_carry;
  int64_t tiles_per_chunk;
};
// planes of at most this many bytes by default (splitd_bwd_workspace_bytes); the caller may give more or less
constexpr size_t kDefaultPlaneLimit = static_cast<size_t>(9) << 30;

int launch_fwd(const splitd_params* p, cudaStream_t stream);
size_t fwd_workspace_bytes(const splitd_params* p);
int launch_bwd_preprocess(const splitd_params* p, cudaStream_t stream);
// stages: bit 0 = P / dS tiles of chunk `chunk`, bit 1 = dK and dV, bit 2 = dQ from them
int launch_bwd_chunk(const splitd_params* p, const BwdPlan& pl, int chunk, int stages, cudaStream_t stream);
int launch_bwd_pds(const splitd_params* p, const BwdPlan& pl, int chunk, cudaStream_t stream);
int launch_bwd_grad(const splitd_params* p, const BwdPlan& pl, int chunk, cudaStream_t stream, int modes);
size_t bwd_rowstat_elems(const splitd_params* p);
// The optional low word of the output (splitd_params::o_resid): a flag byte per output row (indexed like lse),
// padded to 256 bytes, then one 512-element row per output row.
inline size_t out_resid_flag_bytes(const splitd_params* p) { return (bwd_rowstat_elems(p) + 255) / 256 * 256; }
inline size_t out_resid_bytes(const splitd_params* p) {
  return out_resid_flag_bytes(p) + bwd_rowstat_elems(p) * static_cast<size_t>(kHeadDim) * 2;
}
size_t bwd_workspace_bytes(const splitd_params* p);
size_t bwd_workspace_bytes_full(const splitd_params* p);
size_t bwd_workspace_bytes_for(const splitd_params* p, size_t plane_limit);
int plan_bwd(const splitd_params* p, BwdPlan& pl);
void plan_chunk(const BwdPlan& pl, int i, const splitd_params* p, BwdParams& bp);
int fill_bwd_params(const splitd_params* p, BwdParams& bp, const BwdPlan* pl);
int check_common(const splitd_params* p, bool backward);
int check_device();
void clear_error();

// Number of 2-CTA clusters of `kern` the current device keeps resident at once (the grid of a persistent
// kernel). `cache` holds one entry per device index and is filled on first use, which is also where the kernel's
// dynamic shared memory limit is raised (once per device instead of once per launch). Concurrent first calls
// compute the same value twice; the atomics only make that well defined. Returns <= 0 after a CUDA error.
template <typename Kernel>
inline int resident_cluster_pairs(Kernel kern, int threads, int smem_bytes, std::atomic<int> (&cache)[64]) {
  int dev = 0, resident = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64) {
    const int c = cache[dev].load(std::memory_order_acquire);
    if (c > 0) return c;
  }
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2);
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem_bytes;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  cudaError_t ce = cudaOccupancyMaxActiveClusters(&resident, kern, &cfg);
  if (ce != cudaSuccess || resident <= 0) {
    cudaGetLastError();
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    resident = sms > 1 ? sms / 2 : 1;
  }
  if (dev >= 0 && dev < 64) cache[dev].store(resident, std::memory_order_release);
  return resident;
}

}  // namespace sd
