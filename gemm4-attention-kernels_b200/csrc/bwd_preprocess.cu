// Backward step 1 (HBM-bound), two small kernels:
//  * splitd_bwd_rowmax_kernel reads dO and V once and leaves, per (batch or packed sequence, KV head), the largest
//    |dO row|^2, |dO element| and |V row|^2 in the workspace head. They fix the power-of-two scales of the fp16
//    data the tensor-core kernels exchange (bwd_common.cuh) before anything is converted.
//  * splitd_bwd_preprocess_kernel computes, per query row, dpsum = sum_d O*dO - dLSE and lse_log2 = LSE*log2(e):
//    the quantities of the reference's preprocess kernel (src/flash_bwd_preprocess.py:289-315); rows without
//    keys (LSE = -inf) get lse_log2 = 0 so that exp2(masked score - 0) is still 0 (:252-254). On the way it
//    writes the fp16 copies of dO (scaled) and Q, records the largest |dpsum| per group, and a second group of
//    blocks copies K to fp16.
// One warp per (token, head) row: 2 x 16-byte loads per lane and tensor, shuffle reduction.
// Also hosts the helpers that size, lay out and chunk the backward workspace.
#include <cstring>

#include "bwd_common.cuh"
#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"
#include "rowcopy.cuh"

namespace sd {

namespace pre {
constexpr int kTokensPerBlock = 64;  // 8 warps x 8 tokens
}

// sequence that holds packed token `tok` (cu has n + 1 non-decreasing entries, cu[0] = 0)
__device__ __forceinline__ int find_sequence(const int* cu, int n, int tok) {
  int lo = 0, hi = n;  // invariant: cu[lo] <= tok < cu[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu[mid] <= tok) lo = mid; else hi = mid;
  }
  return lo;
}

// Block -> (part, batch, KV head, 64-token chunk); every warp takes 8 of the tokens. Part 0 walks the query
// tokens (and there the query heads of the KV head), part 1 the key tokens.
struct PreBlock {
  bool k_part, packed;
  int chunk, kvh, b_blk, n_tok;
  const int* cu;
};
__device__ __forceinline__ PreBlock pre_block(const BwdParams& p, int q_blocks, int q_chunks, int k_chunks) {
  const TileGeom& g = p.g;
  PreBlock pb;
  pb.packed = g.cu_q != nullptr;
  pb.k_part = static_cast<int>(blockIdx.x) >= q_blocks;
  int blk = pb.k_part ? blockIdx.x - q_blocks : blockIdx.x;
  const int chunks = pb.k_part ? k_chunks : q_chunks;
  pb.chunk = blk % chunks;
  blk /= chunks;
  pb.kvh = blk % g.heads_kv;
  pb.b_blk = blk / g.heads_kv;  // batched layout: the batch; packed: 0
  pb.n_tok = pb.packed ? (pb.k_part ? p.total_k : p.total_q) : (pb.k_part ? g.seqlen_k : g.seqlen_q);
  pb.cu = pb.k_part ? g.cu_k : g.cu_q;
  return pb;
}

__global__ void __launch_bounds__(256) splitd_bwd_rowmax_kernel(const BwdParams p, int q_blocks, int q_chunks,
                                                                int k_chunks) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const TileGeom& g = p.g;
  const PreBlock pb = pre_block(p, q_blocks, q_chunks, k_chunks);
  int cur_grp = -1;
  float m_n2 = 0.f, m_el = 0.f;  // running maxima of the current group: |row|^2, |element|
  auto flush = [&]() {
    if (cur_grp >= 0 && lane == 0) {
      uint32_t* st = p.stats + static_cast<int64_t>(cur_grp) * kStatWords;
      if (pb.k_part) {
        atomicMax(st + kStatV2, __float_as_uint(m_n2));
      } else {
        atomicMax(st + kStatDo2, __float_as_uint(m_n2));
        atomicMax(st + kStatDoMax, __float_as_uint(m_el));
      }
    }
    m_n2 = 0.f, m_el = 0.f;
  };
  for (int i = 0; i < 8; ++i) {
    const int tok = pb.chunk * pre::kTokensPerBlock + i * 8 + warp;
    if (tok >= pb.n_tok) break;
    const int b = pb.packed ? find_sequence(pb.cu, g.batch, tok) : pb.b_blk;
    const int grp = b * g.heads_kv + pb.kvh;
    if (grp != cur_grp) {
      flush();
      cur_grp = grp;
    }
    const int n_rows = pb.k_part ? 1 : g.group;
    for (int hg = 0; hg < n_rows; ++hg) {
      const uint16_t* r;
      if (pb.k_part)
        r = reinterpret_cast<const uint16_t*>(p.v) + (pb.packed ? 0 : b * p.v_stride_b) +
            static_cast<int64_t>(tok) * p.v_stride_s + pb.kvh * p.v_stride_h;
      else
        r = reinterpret_cast<const uint16_t*>(p.dout) + (pb.packed ? 0 : b * p.do_stride_b) +
            static_cast<int64_t>(tok) * p.do_stride_s + (pb.kvh * g.group + hg) * p.do_stride_h;
      const Row16 v = load_row(r, lane);
      float n2 = 0.f, el = 0.f;
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        n2 = fmaf(v.x[e], v.x[e], n2);
        el = fmaxf(el, fabsf(v.x[e]));
      }
      m_n2 = fmaxf(m_n2, warp_sum(n2));
      m_el = fmaxf(m_el, warp_max(el));
    }
  }
  flush();
}

__global__ void __launch_bounds__(256, 3) splitd_bwd_preprocess_kernel(const BwdParams p, int q_blocks, int q_chunks,
                                                                    int k_chunks) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const TileGeom& g = p.g;
  const PreBlock pb = pre_block(p, q_blocks, q_chunks, k_chunks);
  int cur_grp = -1;
  float m_delta = 0.f, do_mul = 1.f;
  auto flush = [&]() {
    if (cur_grp >= 0 && lane == 0 && !pb.k_part)
      atomicMax(p.stats + static_cast<int64_t>(cur_grp) * kStatWords + kStatDelta, __float_as_uint(m_delta));
    m_delta = 0.f;
  };
  for (int i = 0; i < 8; ++i) {
    const int tok = pb.chunk * pre::kTokensPerBlock + i * 8 + warp;
    if (tok >= pb.n_tok) break;
    const int b = pb.packed ? find_sequence(pb.cu, g.batch, tok) : pb.b_blk;
    if (pb.k_part) {
      const uint16_t* kr = reinterpret_cast<const uint16_t*>(p.k) + (pb.packed ? 0 : b * p.k_stride_b) +
                           static_cast<int64_t>(tok) * p.k_stride_s + pb.kvh * p.k_stride_h;
      const int64_t row = (static_cast<int64_t>(pb.packed ? 0 : b) * pb.n_tok + tok) * g.heads_kv + pb.kvh;
      store_row_half(p.k_h + row * kHeadDim, lane, load_row(kr, lane), 1.f);
      continue;
    }
    const int grp = b * g.heads_kv + pb.kvh;
    if (grp != cur_grp) {
      flush();
      cur_grp = grp;
      do_mul = pow2i(do_exponent(p.stats + static_cast<int64_t>(grp) * kStatWords));
    }
    for (int hg = 0; hg < g.group; ++hg) {
      const int head = pb.kvh * g.group + hg;
      const int64_t bo = pb.packed ? 0 : b;
      Row16 o = load_row(reinterpret_cast<const uint16_t*>(p.o) + bo * p.o_stride_b +
                             static_cast<int64_t>(tok) * p.o_stride_s + head * p.o_stride_h, lane);
      const Row16 d = load_row(reinterpret_cast<const uint16_t*>(p.dout) + bo * p.do_stride_b +
                                   static_cast<int64_t>(tok) * p.do_stride_s + head * p.do_stride_h, lane);
      const Row16 qr = load_row(reinterpret_cast<const uint16_t*>(p.q) + bo * p.q_stride_b +
                                    static_cast<int64_t>(tok) * p.q_stride_s + head * p.q_stride_h, lane);
      const int64_t row = (bo * pb.n_tok + tok) * g.heads_q + head;  // contiguous (B,S,H,512) / (T,H,512) copies
      const int64_t idx = pb.packed ? static_cast<int64_t>(head) * p.total_q + tok
                                    : (static_cast<int64_t>(b) * g.heads_q + head) * g.seqlen_q + tok;
      if (p.resid_rows != nullptr && p.resid_flags[idx] != 0) {  // the low word the forward kept of this row
        const Row16 lo = load_row(p.resid_rows + row * kHeadDim, lane);
#pragma unroll
        for (int e = 0; e < 16; ++e) o.x[e] += lo.x[e];
      }
      store_row_half(p.do_h + row * kHeadDim, lane, d, do_mul);
      store_row_half(p.q_h + row * kHeadDim, lane, qr, 1.f);
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < 16; ++e) acc = fmaf(o.x[e], d.x[e], acc);
      acc = warp_sum(acc);
      if (p.dlse) acc -= p.dlse[idx];
      if (lane == 0) {
        const float l = p.lse[idx];
        p.dpsum[idx] = acc;
        p.lse_log2[idx] = (l == -INFINITY) ? 0.f : l * kLog2e;
      }
      m_delta = fmaxf(m_delta, fabsf(acc));
    }
  }
  flush();
}

static inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

size_t bwd_rowstat_elems(const splitd_params* p) {
  const bool varlen = p->cu_seqlens_q != nullptr;
  return varlen ? static_cast<size_t>(p->heads_q) * p->total_q
                : static_cast<size_t>(p->batch) * p->heads_q * p->seqlen_q;
}

// ---------------------------------------------------------------------------------------------------------
// workspace layout and chunk plan
// ---------------------------------------------------------------------------------------------------------
static bool plan_shape(const splitd_params* p, BwdPlan& pl) {
  if (p->heads_kv <= 0 || p->heads_q <= 0 || p->heads_q % p->heads_kv || p->batch <= 0) return false;
  TileGeom g;
  fill_geom(p, g);
  const bool varlen = p->cu_seqlens_q != nullptr;
  memset(&pl, 0, sizeof(pl));
  pl.head_units = g.head_units;
  pl.upk = g.head_units / p->heads_kv;
  pl.row_tiles_seq = varlen ? 0 : g.row_tiles;
  pl.batch = p->batch;
  pl.g_end = varlen ? g.row_tiles : static_cast<int64_t>(g.row_tiles) * g.batch;
  // +64 elements (one 128-byte line) so consecutive rows do not sit a power of two apart in HBM
  pl.pitch = round_up(varlen ? (p->max_seqlen_k < p->total_k ? p->max_seqlen_k : p->total_k) : p->seqlen_k, 256) + 64;
  pl.tile_bytes = static_cast<size_t>(2) * kRowsPerPair * pl.pitch * sizeof(uint16_t);
  pl.head_bytes = static_cast<size_t>(
      round_up(kWsCounterBytes + static_cast<int64_t>(p->batch) * p->heads_kv * kStatWords * 4, 256));
  const int64_t tok_q = varlen ? p->total_q : static_cast<int64_t>(p->batch) * p->seqlen_q;
  const int64_t tok_k = varlen ? p->total_k : static_cast<int64_t>(p->batch) * p->seqlen_k;
  pl.copy_q_bytes = static_cast<size_t>(round_up(tok_q * p->heads_q * kHeadDim * 2, 256));   // each of dO_h, Q_h
  pl.copy_k_bytes = static_cast<size_t>(round_up(tok_k * p->heads_kv * kHeadDim * 2, 256));
  pl.fixed_bytes = pl.head_bytes + 2 * pl.copy_q_bytes + pl.copy_k_bytes;
  const int64_t key_tiles = varlen ? (p->total_k / 256 + p->batch) : static_cast<int64_t>(p->batch) * ((p->seqlen_k + 255) / 256);
  pl.carry_bytes = static_cast<size_t>(key_tiles) * 2 * 2 * kRowsPerPair * kHeadDim * sizeof(float);
  pl.full_bytes = static_cast<size_t>(pl.head_units) * pl.g_end * pl.tile_bytes;
  return true;
}

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Chooses how the (head unit) x (row tile) space is cut so that the planes of one chunk fit `avail` bytes.
// Returns false when even the smallest chunk does not fit.
static bool plan_chunks(BwdPlan& pl, size_t avail_total) {
  if (avail_total < pl.fixed_bytes) return false;
  const size_t avail = avail_total - pl.fixed_bytes;
  const int heads_kv = pl.head_units / pl.upk;
  const size_t kv_bytes = static_cast<size_t>(pl.upk) * pl.g_end * pl.tile_bytes;
  pl.use_carry = 0;
  if (avail >= pl.full_bytes) {  // everything at once
    pl.mode = 0, pl.n_chunks = 1;
    return true;
  }
  if (avail >= kv_bytes) {  // whole KV heads
    const int64_t fit = avail / kv_bytes;
    pl.mode = 1;
    pl.n_chunks = static_cast<int>(ceil_div(heads_kv, fit));
    pl.kv_per_chunk = static_cast<int>(ceil_div(heads_kv, pl.n_chunks));
    return true;
  }
  const size_t kvb_bytes = static_cast<size_t>(pl.upk) * pl.row_tiles_seq * pl.tile_bytes;  // one KV head, one batch
  if (pl.row_tiles_seq > 0 && kvb_bytes > 0 && avail >= kvb_bytes) {
    const int64_t fit = avail / kvb_bytes;
    pl.mode = 2;
    pl.slices = static_cast<int>(ceil_div(pl.batch, fit));
    pl.batches_per_chunk = static_cast<int>(ceil_div(pl.batch, pl.slices));
    pl.n_chunks = heads_kv * pl.slices;
    return true;
  }
  // one head unit at a time, its row tiles in ranges; dK / dV accumulators travel between the chunks
  if (avail < pl.carry_bytes + 3 * pl.tile_bytes) return false;
  int64_t fit = static_cast<int64_t>((avail - pl.carry_bytes) / pl.tile_bytes) - 1;  // one tile of slack, see plan_chunk
  fit &= ~static_cast<int64_t>(1);
  pl.mode = 3, pl.use_carry = 1;
  pl.slices = static_cast<int>(ceil_div(pl.g_end, fit));
  pl.tiles_per_chunk = (ceil_div(pl.g_end, pl.slices) + 1) & ~static_cast<int64_t>(1);
  pl.slices = static_cast<int>(ceil_div(pl.g_end, pl.tiles_per_chunk));
  pl.n_chunks = pl.head_units * pl.slices;
  return true;
}

size_t bwd_workspace_bytes_for(const splitd_params* p, size_t plane_limit) {
  BwdPlan pl;
  if (!plan_shape(p, pl)) return 0;
  if (pl.full_bytes <= plane_limit) return pl.fixed_bytes + pl.full_bytes;
  const size_t kv_bytes = static_cast<size_t>(pl.upk) * pl.g_end * pl.tile_bytes;
  if (kv_bytes <= plane_limit) return pl.fixed_bytes + plane_limit / kv_bytes * kv_bytes;
  const size_t kvb_bytes = static_cast<size_t>(pl.upk) * pl.row_tiles_seq * pl.tile_bytes;
  if (pl.row_tiles_seq > 0 && kvb_bytes <= plane_limit) return pl.fixed_bytes + plane_limit / kvb_bytes * kvb_bytes;
  size_t tiles = plane_limit / pl.tile_bytes;
  if (tiles < 3) tiles = 3;
  return pl.fixed_bytes + pl.carry_bytes + tiles * pl.tile_bytes;
}

size_t bwd_workspace_bytes(const splitd_params* p) { return bwd_workspace_bytes_for(p, kDefaultPlaneLimit); }
size_t bwd_workspace_bytes_full(const splitd_params* p) { return bwd_workspace_bytes_for(p, ~static_cast<size_t>(0) >> 1); }

int plan_bwd(const splitd_params* p, BwdPlan& pl) {
  if (!plan_shape(p, pl)) return fail(SPLITD_ERR_INVALID_ARGUMENT, "bad head counts or batch");
  if (!p->workspace) return fail(SPLITD_ERR_WORKSPACE, "workspace is NULL (%zu bytes required)", bwd_workspace_bytes(p));
  if (reinterpret_cast<uintptr_t>(p->workspace) % 256 != 0)
    return fail(SPLITD_ERR_WORKSPACE, "workspace must be 256-byte aligned");
  if (!plan_chunks(pl, p->workspace_bytes))
    return fail(SPLITD_ERR_WORKSPACE, "workspace of at least %zu bytes required (%zu recommended), got %zu",
                bwd_workspace_bytes_for(p, 0), bwd_workspace_bytes(p), p->workspace_bytes);
  return 0;
}

// Chunk i of the plan, in the order the accumulation of dK / dV needs: head units ascending, row tiles descending.
void plan_chunk(const BwdPlan& pl, int i, const splitd_params* p, BwdParams& bp) {
  int64_t hu0 = 0, hu1 = pl.head_units, g0 = 0, g1 = pl.g_end;
  if (pl.mode == 1) {
    hu0 = static_cast<int64_t>(i) * pl.kv_per_chunk * pl.upk;
    hu1 = hu0 + static_cast<int64_t>(pl.kv_per_chunk) * pl.upk;
  } else if (pl.mode == 2) {
    const int kv = i / pl.slices, sl = pl.slices - 1 - i % pl.slices;
    hu0 = static_cast<int64_t>(kv) * pl.upk, hu1 = hu0 + pl.upk;
    g0 = static_cast<int64_t>(sl) * pl.batches_per_chunk * pl.row_tiles_seq;
    g1 = g0 + static_cast<int64_t>(pl.batches_per_chunk) * pl.row_tiles_seq;
  } else if (pl.mode == 3) {
    const int sl = pl.slices - 1 - i % pl.slices;
    hu0 = i / pl.slices, hu1 = hu0 + 1;
    g0 = sl * pl.tiles_per_chunk, g1 = g0 + pl.tiles_per_chunk;
  }
  if (hu1 > pl.head_units) hu1 = pl.head_units;
  if (g1 > pl.g_end) g1 = pl.g_end;
  bp.c_hu0 = static_cast<int>(hu0), bp.c_hu1 = static_cast<int>(hu1);
  bp.c_g0 = static_cast<int>(g0), bp.c_g1 = static_cast<int>(g1);
  bp.carry_mode = pl.use_carry;
  // row ranges cut anywhere (mode 3): a pair that starts on the last tile of the range brings its second tile
  // along, hence one tile of slack. Ranges that end with a sequence (the other modes) never split a pair.
  bp.ws_rows = ((pl.mode == 3 && g1 < pl.g_end ? g1 + 1 : g1) - g0) * kRowsPerPair;
  bp.c_b0 = 0, bp.c_nb = 1;
  const int ppu_seq = (pl.row_tiles_seq + 1) / 2;
  bp.c_tp0 = 0, bp.c_ntp = ppu_seq;
  if (pl.row_tiles_seq > 0) {
    const int b_lo = static_cast<int>(g0 / pl.row_tiles_seq), b_hi = static_cast<int>((g1 - 1) / pl.row_tiles_seq);
    bp.c_b0 = b_lo, bp.c_nb = b_hi - b_lo + 1;
    if (bp.c_nb == 1) {
      const int64_t tb = static_cast<int64_t>(b_lo) * pl.row_tiles_seq;
      const int64_t lo = (g0 - tb + 1) / 2, hi = (g1 - tb + 1) / 2;
      bp.c_tp0 = static_cast<int>(lo);
      bp.c_ntp = static_cast<int>((hi < ppu_seq ? hi : ppu_seq) - lo);
    }
  }
  (void)p;
}

int fill_bwd_params(const splitd_params* p, BwdParams& bp, const BwdPlan* pl) {
  memset(&bp, 0, sizeof(bp));
  fill_geom(p, bp.g);
  bp.lse = p->lse;
  bp.dlse = p->dlse;
  bp.dpsum = p->dpsum;
  bp.lse_log2 = p->lse_log2;
  bp.o = p->o;
  bp.resid_flags = static_cast<const uint8_t*>(p->o_resid);
  bp.resid_rows = p->o_resid ? reinterpret_cast<const uint16_t*>(static_cast<const uint8_t*>(p->o_resid) +
                                                                 out_resid_flag_bytes(p))
                             : nullptr;
  bp.dout = p->dout;
  bp.q = p->q;
  bp.k = p->k;
  bp.v = p->v;
  bp.dq = p->dq;
  bp.dk = p->dk;
  bp.dv = p->dv;
  bp.o_stride_b = p->o_strides[0], bp.o_stride_s = p->o_strides[1], bp.o_stride_h = p->o_strides[2];
  bp.do_stride_b = p->do_strides[0], bp.do_stride_s = p->do_strides[1], bp.do_stride_h = p->do_strides[2];
  bp.q_stride_b = p->q_strides[0], bp.q_stride_s = p->q_strides[1], bp.q_stride_h = p->q_strides[2];
  bp.k_stride_b = p->k_strides[0], bp.k_stride_s = p->k_strides[1], bp.k_stride_h = p->k_strides[2];
  bp.v_stride_b = p->v_strides[0], bp.v_stride_s = p->v_strides[1], bp.v_stride_h = p->v_strides[2];
  bp.dq_stride_b = p->dq_strides[0], bp.dq_stride_s = p->dq_strides[1], bp.dq_stride_h = p->dq_strides[2];
  bp.dk_stride_b = p->dk_strides[0], bp.dk_stride_s = p->dk_strides[1], bp.dk_stride_h = p->dk_strides[2];
  bp.dv_stride_b = p->dv_strides[0], bp.dv_stride_s = p->dv_strides[1], bp.dv_stride_h = p->dv_strides[2];
  const int64_t* all[8] = {p->o_strides, p->do_strides, p->dq_strides, p->dk_strides,
                           p->dv_strides, p->q_strides,  p->k_strides,  p->v_strides};
  for (auto st : all)
    for (int i = 0; i < 3; ++i)
      if (st[i] % 8 != 0) return fail(SPLITD_ERR_INVALID_ARGUMENT, "tensor strides must be multiples of 8 elements");
  const void* ptrs[8] = {p->o, p->dout, p->dq, p->dk, p->dv, p->q, p->k, p->v};
  for (auto q : ptrs)
    if (reinterpret_cast<uintptr_t>(q) % 16 != 0)
      return fail(SPLITD_ERR_INVALID_ARGUMENT, "q/k/v/o/dout/dq/dk/dv must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(p->o_resid) % 256 != 0)
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "o_resid must be 256-byte aligned");
  bp.total_q = p->total_q;
  bp.total_k = p->total_k;
  const bool varlen = p->cu_seqlens_q != nullptr;
  bp.key_tiles = varlen ? (p->total_k / 256 + p->batch) : (p->seqlen_k + 255) / 256;
  bp.scale = p->softmax_scale;
  bp.scale_log2 = p->softmax_scale * kLog2e;
  bp.status = p->status_flag;
  bp.debug = p->debug;
  if (pl) {
    uint8_t* base = static_cast<uint8_t*>(p->workspace);
    bp.tile_counters = reinterpret_cast<int*>(base);
    bp.stats = reinterpret_cast<uint32_t*>(base + kWsCounterBytes);
    bp.do_h = reinterpret_cast<uint16_t*>(base + pl->head_bytes);
    bp.q_h = reinterpret_cast<uint16_t*>(base + pl->head_bytes + pl->copy_q_bytes);
    bp.k_h = reinterpret_cast<uint16_t*>(base + pl->head_bytes + 2 * pl->copy_q_bytes);
    bp.carry = pl->use_carry ? reinterpret_cast<float*>(base + pl->fixed_bytes) : nullptr;
    bp.ws = reinterpret_cast<uint16_t*>(base + pl->fixed_bytes + (pl->use_carry ? pl->carry_bytes : 0));
    bp.ws_pitch = pl->pitch;
    bp.g_end = static_cast<int>(pl->g_end);
  }
  return 0;
}

int launch_bwd_preprocess(const splitd_params* p, cudaStream_t stream) {
  BwdPlan pl;
  if (int e = plan_bwd(p, pl)) return e;
  BwdParams bp;
  if (int e = fill_bwd_params(p, bp, &pl)) return e;
  const bool varlen = p->cu_seqlens_q != nullptr;
  const int64_t q_chunks = ((varlen ? p->total_q : p->seqlen_q) + pre::kTokensPerBlock - 1) / pre::kTokensPerBlock;
  const int64_t k_chunks = ((varlen ? p->total_k : p->seqlen_k) + pre::kTokensPerBlock - 1) / pre::kTokensPerBlock;
  const int64_t groups = static_cast<int64_t>(p->heads_kv) * (varlen ? 1 : p->batch);
  const int64_t q_blocks = q_chunks * groups, blocks = q_blocks + k_chunks * groups;
  if (blocks <= 0 || blocks > 0x7fffffffll) return fail(SPLITD_ERR_INVALID_ARGUMENT, "preprocess grid out of range");
  // work counters and the maxima start at zero
  cudaError_t ce = cudaMemsetAsync(p->workspace, 0, pl.head_bytes, stream);
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "cudaMemsetAsync(workspace head): %s", cudaGetErrorString(ce));
  splitd_bwd_rowmax_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      bp, static_cast<int>(q_blocks), static_cast<int>(q_chunks), static_cast<int>(k_chunks));
  splitd_bwd_preprocess_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      bp, static_cast<int>(q_blocks), static_cast<int>(q_chunks), static_cast<int>(k_chunks));
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "preprocess launch failed: %s", cudaGetErrorString(ce));
  return 0;
}

}  // namespace sd
