// C-ABI entry points (see include/splitd_attn.h): argument validation, TMA descriptor
// construction, launch configuration. No device allocation, no synchronisation.
#include <cudaTypedefs.h>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include <atomic>

#include "../../include/splitd_attn.h"
#include "common.cuh"
#include "launch.cuh"

namespace sd {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

void clear_error() { g_err[0] = 0; }

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static std::atomic<PFN_cuTensorMapEncodeTiled_v12000> cached{nullptr};
  if (auto fn = cached.load(std::memory_order_acquire)) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  auto fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  cached.store(fn, std::memory_order_release);
  return fn;
}

// 16-bit elements, 128-byte swizzle, innermost box = 64 elements.
int make_tmap(CUtensorMap* map, const void* base, int rank, const uint64_t* dims, const int64_t* strides_elems,
              const uint32_t* box, const char* what) {
  auto fn = encode_fn();
  if (!fn) return fail(SPLITD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  cuuint64_t gdim[5];
  cuuint64_t gstride[4];
  cuuint32_t gbox[5], estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      if (strides_elems[i] <= 0 || (strides_elems[i] * 2) % 16 != 0)
        return fail(SPLITD_ERR_INVALID_ARGUMENT, "%s: stride %lld of dim %d must be a positive multiple of 8 elements",
                    what, (long long)strides_elems[i], i);
      gstride[i - 1] = static_cast<cuuint64_t>(strides_elems[i]) * 2;
    }
  }
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0)
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "%s: base pointer must be 16-byte aligned", what);
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, rank, const_cast<void*>(base), gdim, gstride, gbox, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SPLITD_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, (int)r);
  return 0;
}

int check_common(const splitd_params* p, bool backward) {
  if (!p) return fail(SPLITD_ERR_INVALID_ARGUMENT, "params is NULL");
  if (!p->q || !p->k || !p->v || !p->o) return fail(SPLITD_ERR_INVALID_ARGUMENT, "q, k, v and o must not be NULL");
  if (p->head_dim != kHeadDim)
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "head_dim == 512 is required, got %d", p->head_dim);
  if (p->heads_q <= 0 || p->heads_kv <= 0 || p->heads_q % p->heads_kv != 0)
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "heads_q (%d) must be a positive multiple of heads_kv (%d)", p->heads_q,
                p->heads_kv);
  if (p->dtype != SPLITD_DTYPE_BF16 && p->dtype != SPLITD_DTYPE_FP16)
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "dtype must be SPLITD_DTYPE_BF16 or SPLITD_DTYPE_FP16");
  if (!(p->softmax_scale > 0.f)) return fail(SPLITD_ERR_INVALID_ARGUMENT, "softmax_scale must be > 0");
  if (p->batch <= 0) return fail(SPLITD_ERR_INVALID_ARGUMENT, "batch must be > 0");
  const bool varlen = p->cu_seqlens_q != nullptr || p->cu_seqlens_k != nullptr;
  if (varlen) {
    if (!p->cu_seqlens_q || !p->cu_seqlens_k)
      return fail(SPLITD_ERR_INVALID_ARGUMENT, "cu_seqlens_q and cu_seqlens_k must be given together");
    if (p->total_q <= 0 || p->total_k <= 0 || p->max_seqlen_q <= 0 || p->max_seqlen_k <= 0)
      return fail(SPLITD_ERR_INVALID_ARGUMENT, "packed layout needs total_q/k and max_seqlen_q/k > 0");
  } else if (p->seqlen_q <= 0 || p->seqlen_k <= 0) {
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "seqlen_q and seqlen_k must be > 0");
  }
  if (p->softcap < 0.f) return fail(SPLITD_ERR_INVALID_ARGUMENT, "softcap must be >= 0");
  if (p->local && (p->window_left < -1 || p->window_right < -1))
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "window_left / window_right must be >= -1");
  if (p->causal && p->local)
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "causal and a sliding window are mutually exclusive");
  if (backward) {
    if (p->softcap > 0.f || p->local)
      return fail(SPLITD_ERR_UNSUPPORTED, "backward does not support softcap or sliding windows");
    if (p->dtype != SPLITD_DTYPE_BF16)
      return fail(SPLITD_ERR_UNSUPPORTED, "backward supports bfloat16 only");
    if (!p->dout || !p->dq || !p->dk || !p->dv || !p->lse || !p->dpsum || !p->lse_log2)
      return fail(SPLITD_ERR_INVALID_ARGUMENT, "dout, dq, dk, dv, lse, dpsum and lse_log2 must not be NULL");
  }
  return 0;
}

int check_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(SPLITD_ERR_CUDA, "cudaGetDevice failed");
  int s = splitd_device_supported(dev);
  if (s < 0) return s;
  if (s == 0) return fail(SPLITD_ERR_DEVICE, "device %d is not compute capability 10.x", dev);
  return 0;
}

// Heads are folded into rows when the group size divides the 64 rows one CTA owns.
void fill_geom(const splitd_params* p, TileGeom& g, int rows_per_cta) {
  const bool varlen = p->cu_seqlens_q != nullptr;
  g.batch = p->batch;
  g.seqlen_q = varlen ? p->max_seqlen_q : p->seqlen_q;
  g.seqlen_k = varlen ? p->max_seqlen_k : p->seqlen_k;
  g.heads_q = p->heads_q;
  g.heads_kv = p->heads_kv;
  g.group = p->heads_q / p->heads_kv;
  g.pack_g = (g.group > 1 && g.group <= kRowsPerCta && kRowsPerCta % g.group == 0) ? g.group : 1;
  g.head_units = (g.pack_g == g.group) ? p->heads_kv : p->heads_q;
  g.pos_per_cta = rows_per_cta / g.pack_g;
  g.causal = p->causal ? 1 : 0;
  g.cu_q = p->cu_seqlens_q;
  g.cu_k = p->cu_seqlens_k;
  const int ppp = 2 * g.pos_per_cta;
  g.row_tiles = varlen ? (p->total_q / ppp + p->batch) : (p->seqlen_q + ppp - 1) / ppp;
}

// Q-like tensor (q, dout): dims (D, pack_g, tokens, head_units, batch); box (64, pack_g, pos_per_cta, 1, 1)
int make_q_tmap(CUtensorMap* map, const void* base, const splitd_params* p, const TileGeom& g, const int64_t* st,
                int box_pos, const char* what) {
  const bool varlen = p->cu_seqlens_q != nullptr;
  const uint64_t dims[5] = {kHeadDim, (uint64_t)g.pack_g, (uint64_t)(varlen ? p->total_q : p->seqlen_q),
                            (uint64_t)g.head_units, (uint64_t)(varlen ? 1 : p->batch)};
  const int64_t strides[5] = {1, st[2], st[1], st[2] * g.pack_g, varlen ? st[1] * p->total_q : st[0]};
  const uint32_t box[5] = {64, (uint32_t)g.pack_g, (uint32_t)box_pos, 1, 1};
  return make_tmap(map, base, 5, dims, strides, box, what);
}

// K-like tensor (k, v): dims (D, tokens, heads_kv, batch); box (64, rows, 1, 1)
int make_kv_tmap(CUtensorMap* map, const void* base, const splitd_params* p, const int64_t* st, int box_rows,
                 const char* what) {
  const bool varlen = p->cu_seqlens_k != nullptr;
  const uint64_t dims[4] = {kHeadDim, (uint64_t)(varlen ? p->total_k : p->seqlen_k), (uint64_t)p->heads_kv,
                            (uint64_t)(varlen ? 1 : p->batch)};
  const int64_t strides[4] = {1, st[1], st[2], varlen ? st[1] * p->total_k : st[0]};
  const uint32_t box[4] = {64, (uint32_t)box_rows, 1, 1};
  return make_tmap(map, base, 4, dims, strides, box, what);
}

}  // namespace sd

using namespace sd;

extern "C" {

const char* splitd_last_error(void) { return g_err; }
const char* splitd_version(void) { return "splitd_attn sm_100a 0.1"; }

int splitd_device_supported(int device) {
  int major = 0;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
    cudaGetLastError();
    return fail(SPLITD_ERR_CUDA, "cudaDeviceGetAttribute failed for device %d", device);
  }
  return major == 10 ? 1 : 0;
}

int splitd_fwd(const splitd_params* p, void* stream) {
  g_err[0] = 0;
  if (int e = check_common(p, false)) return e;
  if (int e = check_device()) return e;
  return launch_fwd(p, static_cast<cudaStream_t>(stream));
}

size_t splitd_fwd_workspace_bytes(const splitd_params* p) { return p ? fwd_workspace_bytes(p) : 0; }

size_t splitd_bwd_rowstat_elems(const splitd_params* p) { return p ? bwd_rowstat_elems(p) : 0; }

size_t splitd_out_resid_bytes(const splitd_params* p) { return p ? out_resid_bytes(p) : 0; }
size_t splitd_bwd_workspace_bytes(const splitd_params* p) { return p ? bwd_workspace_bytes(p) : 0; }
size_t splitd_bwd_workspace_bytes_limit(const splitd_params* p, size_t tile_bytes_limit) {
  return p ? bwd_workspace_bytes_for(p, tile_bytes_limit) : 0;
}

static int check_bwd(const splitd_params* p) {
  g_err[0] = 0;
  if (int e = check_common(p, true)) return e;
  return check_device();
}
// the steps that hand P / dS from one call to the next need all of them in the workspace at once
static int plan_single_chunk(const splitd_params* p, BwdPlan& pl, const char* what) {
  if (int e = plan_bwd(p, pl)) return e;
  if (pl.n_chunks != 1)
    return fail(SPLITD_ERR_WORKSPACE,
                "%s keeps the P/dS tiles of the whole problem in the workspace: %zu bytes required, got %zu "
                "(splitd_bwd and splitd_bwd_chunk work with less)",
                what, bwd_workspace_bytes_full(p), p->workspace_bytes);
  return 0;
}

int splitd_bwd_preprocess(const splitd_params* p, void* stream) {
  if (int e = check_bwd(p)) return e;
  return launch_bwd_preprocess(p, static_cast<cudaStream_t>(stream));
}

int splitd_bwd_dq(const splitd_params* p, void* stream) {
  if (int e = check_bwd(p)) return e;
  BwdPlan pl;
  if (int e = plan_single_chunk(p, pl, "splitd_bwd_dq")) return e;
  return launch_bwd_chunk(p, pl, 0, 1 | 4, static_cast<cudaStream_t>(stream));
}

int splitd_bwd_dkdv(const splitd_params* p, void* stream) {
  if (int e = check_bwd(p)) return e;
  BwdPlan pl;
  if (int e = plan_single_chunk(p, pl, "splitd_bwd_dkdv")) return e;
  return launch_bwd_chunk(p, pl, 0, 2, static_cast<cudaStream_t>(stream));
}

int splitd_bwd_tiles(const splitd_params* p, void* stream) {
  if (int e = check_bwd(p)) return e;
  BwdPlan pl;
  if (int e = plan_single_chunk(p, pl, "splitd_bwd_tiles")) return e;
  return launch_bwd_chunk(p, pl, 0, 1, static_cast<cudaStream_t>(stream));
}

int splitd_bwd_grads(const splitd_params* p, void* stream) {
  if (int e = check_bwd(p)) return e;
  BwdPlan pl;
  if (int e = plan_single_chunk(p, pl, "splitd_bwd_grads")) return e;
  return launch_bwd_chunk(p, pl, 0, 2 | 4, static_cast<cudaStream_t>(stream));
}

int splitd_bwd_num_chunks(const splitd_params* p) {
  if (int e = check_bwd(p)) return e;
  BwdPlan pl;
  if (int e = plan_bwd(p, pl)) return e;
  return pl.n_chunks;
}

int splitd_bwd_chunk(const splitd_params* p, int chunk, int stages, void* stream) {
  if (int e = check_bwd(p)) return e;
  BwdPlan pl;
  if (int e = plan_bwd(p, pl)) return e;
  if (chunk < 0 || chunk >= pl.n_chunks) return fail(SPLITD_ERR_INVALID_ARGUMENT, "chunk %d of %d", chunk, pl.n_chunks);
  if (stages != 1 && stages != 2 && stages != 3)
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "stages must be 1 (tiles), 2 (gradients) or 3 (both)");
  return launch_bwd_chunk(p, pl, chunk, (stages & 1) | ((stages & 2) ? 6 : 0), static_cast<cudaStream_t>(stream));
}

int splitd_bwd(const splitd_params* p, void* stream) {
  if (int e = check_bwd(p)) return e;
  BwdPlan pl;
  if (int e = plan_bwd(p, pl)) return e;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (int e = launch_bwd_preprocess(p, s)) return e;
  // per chunk: P/dS tiles, then dQ, dK and dV as one GEMM launch (better tail behaviour than two launches)
  for (int i = 0; i < pl.n_chunks; ++i)
    if (int e = launch_bwd_chunk(p, pl, i, 7, s)) return e;
  return 0;
}

}  // extern "C"
