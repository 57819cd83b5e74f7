// Host-side launchers shared between the C-ABI file and the kernel translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>

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

int launch_fwd(const splitd_params* p, cudaStream_t stream);
int launch_bwd_preprocess(const splitd_params* p, cudaStream_t stream);
int launch_bwd_pds(const splitd_params* p, cudaStream_t stream);
int launch_bwd_pds_two_pass(const splitd_params* p, cudaStream_t stream);
int launch_bwd_grad(const splitd_params* p, cudaStream_t stream, int modes);
int launch_bwd_dq(const splitd_params* p, cudaStream_t stream);
int launch_bwd_dkdv(const splitd_params* p, cudaStream_t stream);
size_t bwd_rowstat_elems(const splitd_params* p);
size_t bwd_workspace_bytes(const splitd_params* p);
int fill_bwd_params(const splitd_params* p, BwdParams& bp);
int check_workspace(const splitd_params* p);

// Number of 2-CTA clusters of `kern` the current device keeps resident at once (the grid of a persistent
// kernel). `cache` holds one entry per device index and is filled on first use.
template <typename Kernel>
inline int resident_cluster_pairs(Kernel kern, int threads, int smem_bytes, int (&cache)[64]) {
  int dev = 0, resident = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && cache[dev] > 0) return cache[dev];
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
  if (dev >= 0 && dev < 64) cache[dev] = resident;
  return resident;
}

}  // namespace sd
