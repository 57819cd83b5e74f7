// Backward step 1 (HBM-bound): per query row, dpsum = sum_d O*dO - dLSE and lse_log2 = LSE*log2(e).
// Same quantities as the reference's preprocess kernel (src/flash_bwd_preprocess.py:289-315); rows
// without keys (LSE = -inf) get lse_log2 = 0 so that exp2(masked score - 0) is still 0 (:252-254).
// One warp per (token, head) row: 2 x 16-byte loads per lane from O and dO, shuffle reduction.
// Also hosts the helpers that size the backward workspace.
#include <cstring>

#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace sd {

__global__ void __launch_bounds__(256) splitd_bwd_preprocess_kernel(const BwdParams p, int64_t n_rows, int tokens_q) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const TileGeom& g = p.g;
  // row -> (b, token, head); heads fastest so consecutive warps read consecutive 1 KB rows
  const int head = static_cast<int>(row % g.heads_q);
  const int64_t tok = row / g.heads_q;  // batched: b * Sq + s ; packed: t
  int b = 0, s = static_cast<int>(tok);
  if (g.cu_q == nullptr) {
    b = static_cast<int>(tok / g.seqlen_q);
    s = static_cast<int>(tok - static_cast<int64_t>(b) * g.seqlen_q);
  }
  const uint16_t* o = reinterpret_cast<const uint16_t*>(p.o) + b * p.o_stride_b + s * p.o_stride_s + head * p.o_stride_h;
  const uint16_t* d = reinterpret_cast<const uint16_t*>(p.dout) + b * p.do_stride_b + s * p.do_stride_s + head * p.do_stride_h;
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + i * 256 + lane * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(d + i * 256 + lane * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, cw[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[t]));
      const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&cw[t]));
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) {
    const int64_t idx = g.cu_q ? static_cast<int64_t>(head) * tokens_q + s
                               : (static_cast<int64_t>(b) * g.heads_q + head) * g.seqlen_q + s;
    const float l = p.lse[idx];
    if (p.dlse) acc -= p.dlse[idx];
    p.dpsum[idx] = acc;
    p.lse_log2[idx] = (l == -INFINITY) ? 0.f : l * kLog2e;
  }
}

static inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

size_t bwd_rowstat_elems(const splitd_params* p) {
  const bool varlen = p->cu_seqlens_q != nullptr;
  return varlen ? static_cast<size_t>(p->heads_q) * p->total_q
                : static_cast<size_t>(p->batch) * p->heads_q * p->seqlen_q;
}

static void ws_shape(const splitd_params* p, const TileGeom& g, int64_t& rows, int64_t& pitch) {
  const bool varlen = p->cu_seqlens_q != nullptr;
  const int64_t tiles = varlen ? g.row_tiles : static_cast<int64_t>(g.row_tiles) * g.batch;
  rows = tiles * kRowsPerPair;
  // +64 elements (one 128-byte line) so consecutive rows do not sit a power of two apart in HBM
  pitch = round_up(varlen ? p->max_seqlen_k : p->seqlen_k, 256) + 64;
}

size_t bwd_workspace_bytes(const splitd_params* p) {
  if (p->heads_kv <= 0 || p->heads_q <= 0 || p->heads_q % p->heads_kv) return 0;
  TileGeom g;
  fill_geom(p, g);
  int64_t rows, pitch;
  ws_shape(p, g, rows, pitch);
  return static_cast<size_t>(2) * g.head_units * rows * pitch * sizeof(uint16_t) + kWsCounterBytes;
}

int fill_bwd_params(const splitd_params* p, BwdParams& bp) {
  memset(&bp, 0, sizeof(bp));
  fill_geom(p, bp.g);
  const TileGeom& g = bp.g;
  bp.lse = p->lse;
  bp.dlse = p->dlse;
  bp.dpsum = p->dpsum;
  bp.lse_log2 = p->lse_log2;
  bp.o = p->o;
  bp.dout = p->dout;
  bp.dq = p->dq;
  bp.dk = p->dk;
  bp.dv = p->dv;
  bp.o_stride_b = p->o_strides[0], bp.o_stride_s = p->o_strides[1], bp.o_stride_h = p->o_strides[2];
  bp.do_stride_b = p->do_strides[0], bp.do_stride_s = p->do_strides[1], bp.do_stride_h = p->do_strides[2];
  bp.dq_stride_b = p->dq_strides[0], bp.dq_stride_s = p->dq_strides[1], bp.dq_stride_h = p->dq_strides[2];
  bp.dk_stride_b = p->dk_strides[0], bp.dk_stride_s = p->dk_strides[1], bp.dk_stride_h = p->dk_strides[2];
  bp.dv_stride_b = p->dv_strides[0], bp.dv_stride_s = p->dv_strides[1], bp.dv_stride_h = p->dv_strides[2];
  const int64_t* all[5] = {p->o_strides, p->do_strides, p->dq_strides, p->dk_strides, p->dv_strides};
  for (auto st : all)
    for (int i = 0; i < 3; ++i)
      if (st[i] % 8 != 0) return fail(SPLITD_ERR_INVALID_ARGUMENT, "o/dout/dq/dk/dv strides must be multiples of 8 elements");
  const void* ptrs[5] = {p->o, p->dout, p->dq, p->dk, p->dv};
  for (auto q : ptrs)
    if (reinterpret_cast<uintptr_t>(q) % 16 != 0)
      return fail(SPLITD_ERR_INVALID_ARGUMENT, "o/dout/dq/dk/dv must be 16-byte aligned");
  bp.ws = reinterpret_cast<uint16_t*>(p->workspace);
  ws_shape(p, g, bp.ws_rows, bp.ws_pitch);
  if (p->workspace)  // the counters sit behind the tiles
    bp.tile_counters = reinterpret_cast<int*>(static_cast<uint8_t*>(p->workspace) +
                                              static_cast<size_t>(2) * g.head_units * bp.ws_rows * bp.ws_pitch * sizeof(uint16_t));
  bp.total_q = p->total_q;
  bp.total_k = p->total_k;
  const bool varlen = p->cu_seqlens_q != nullptr;
  bp.key_tiles = varlen ? (p->total_k / 256 + p->batch) : (p->seqlen_k + 255) / 256;
  bp.scale = p->softmax_scale;
  bp.scale_log2 = p->softmax_scale * kLog2e;
  bp.status = p->status_flag;
  bp.debug = p->debug;
  return 0;
}

int check_workspace(const splitd_params* p) {
  const size_t need = bwd_workspace_bytes(p);
  if (!p->workspace || p->workspace_bytes < need)
    return fail(SPLITD_ERR_WORKSPACE, "workspace of %zu bytes required, got %zu", need, p->workspace_bytes);
  if (reinterpret_cast<uintptr_t>(p->workspace) % 128 != 0)
    return fail(SPLITD_ERR_WORKSPACE, "workspace must be 128-byte aligned");
  return 0;
}

int launch_bwd_preprocess(const splitd_params* p, cudaStream_t stream) {
  BwdParams bp;
  if (int e = fill_bwd_params(p, bp)) return e;
  const bool varlen = p->cu_seqlens_q != nullptr;
  const int64_t tokens = varlen ? p->total_q : static_cast<int64_t>(p->batch) * p->seqlen_q;
  const int64_t n_rows = tokens * p->heads_q;
  const int64_t blocks = (n_rows + 7) / 8;
  if (blocks <= 0 || blocks > 0x7fffffffll) return fail(SPLITD_ERR_INVALID_ARGUMENT, "preprocess grid out of range");
  splitd_bwd_preprocess_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(bp, n_rows, p->total_q);
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "preprocess launch failed: %s", cudaGetErrorString(ce));
  return 0;
}

}  // namespace sd
