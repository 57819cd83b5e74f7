// Backward step 2b / 3: dQ, dK and dV as GEMMs over the fp16 P / dS tiles in the workspace
// (bwd_pds2_kernel.cu), for head_dim 512 on sm_100a.
//
//   dV[keys, 512] = sum over packed rows  P^T  [keys, rows] * dO[rows, 512]
//   dK[keys, 512] = sum over packed rows  dS^T [keys, rows] * Q [rows, 512]
//   dQ[rows, 512] = sum over keys         dS   [rows, keys] * K [keys, 512]
//
// The sums for dK/dV run over ALL query heads of the KV head: with folded heads the packed rows already
// interleave the heads, otherwise the row loop visits each query head of the group. That is the GQA
// reduction the reference does with an in-CTA loop over query heads (src/fmha_dkdv_sm90_d512.py:895-936).
// dQ replaces src/fmha_dq_sm90_d512.py; the math of both is the reference's, only the decomposition is
// different: P and dS are computed once instead of once per D pass per kernel.
//
// One CTA pair owns 256 output rows (keys for dK/dV, packed query rows = two row tiles for dQ) and all
// 512 output columns: cta_group::2 UMMAs with M = 256 (TMEM lane = output row, 128 per CTA), N = 256
// twice, so the fp32 accumulator fills the 512 TMEM columns. Operands stream through a 4 x 48 KB ring:
// per 64-deep contraction chunk, A = 16 KB (this CTA's 128 output rows) and B = 32 KB (this CTA's half
// of the 512 output columns; the pair shares B through the 2-SM MMA).
// Operand forms: P^T / dS^T are read straight from the [rows][keys] workspace as MN-major A; dS for dQ
// is the same memory read as K-major A; dO, Q and K rows are MN-major B. P and dS are fp16 (bwd_common.cuh) and
// the two operands of one MMA must share a format, so B comes from the fp16 copies of dO, Q and K that the
// preprocess step leaves in the workspace. The power-of-two scales of P, dS and dO are taken out of the fp32
// accumulators before the final rounding to bf16.
//
// Persistent pairs: the grid is one pair per SM pair, each drawing output tiles (dV/dK tiles first, then
// dQ tiles, heaviest first) from a global counter (tile_queue.cuh). The producer keeps streaming the next tile's
// operands while the epilogue warps drain the accumulator, and nothing is re-initialised between tiles.
//
// Chunks. One launch covers the head units and row tiles whose P / dS planes the workspace currently holds
// (BwdParams::c_*). A dQ tile only needs its own rows, so it is complete within its chunk. A dK / dV tile sums
// over all rows of its sequence; when a chunk holds only part of them (carry_mode), the tile starts from the
// fp32 accumulator the previous chunk left in `carry` (loaded into TMEM by the epilogue warps before the first
// MMA) and leaves its own there unless it is the last. Chunks run head units ascending and row tiles
// descending, which is the order of the contraction in a single launch, so the result is bit-identical.
#include <cstring>

#include "bwd_common.cuh"
#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"
#include "tile_queue.cuh"

namespace sd {

namespace grad {
constexpr int kStages = 4;
constexpr int kStageBytes = 49152;  // A: 2 x 8 KB, B: 4 x 8 KB
constexpr int kOffCtrl = kStages * kStageBytes;
constexpr int kBarFull = 0;
constexpr int kBarEmpty = 8 * kStages;
constexpr int kBarAccDone = kBarEmpty + 8 * kStages;
constexpr int kBarAccFree = kBarAccDone + 8;
constexpr int kTmemPtr = kBarAccFree + 8;
constexpr int kAbort = kTmemPtr + 4;
constexpr int kTileQ = kAbort + 4;  // TileQueue, kTileQueueBytes
constexpr int kConsumers = 2 + 1 + 16;  // producers, MMA issuer, epilogue warps of both CTAs
constexpr int kCtrlBytes = 256;
constexpr int kSmemBytes = kOffCtrl + kCtrlBytes;
constexpr int kThreads = 384;  // producer, MMA issuer, scheduler, 1 idle warp, 8 epilogue warps
enum { kModeDV = 0, kModeDK = 1, kModeDQ = 2 };
}  // namespace grad

struct GradLaunch {
  int n_kv_pairs;         // tile slots producing dV / dK (even: dV, odd: dK)
  int n_dq_pairs;         // tile slots producing dQ
  int dq_pairs_per_unit;  // packed layout: upper bound of dQ tiles per head unit
  int kv0, kv1;           // KV heads the chunk touches
};

// One output tile of a CTA pair.
struct GradTile {
  int mode, b, sq, sk, q_off, k_off, tile_base, n_row_tiles;
  int kvh, kt;        // dK/dV: kv head, key tile (256 keys)
  int hu, tp;         // dQ: head unit, tile pair
  int u_lo, u_hi;     // dK/dV: query heads of the group summed in this chunk (unfolded groups; else 0, 1)
  int r_lo, r_hi;     // dK/dV: row tiles summed in this chunk
  int kv_tile;        // dK/dV: index of the key tile over all sequences (slot of its travelling accumulator)
  int carry_in, carry_out;
  int n_stages;
};

// Decode tile slot `idx` of the launch. Returns false when the slot holds no tile for this chunk.
__device__ __forceinline__ bool grad_decode(const BwdParams& p, const GradLaunch& gl, int idx, GradTile& t) {
  const TileGeom& g = p.g;
  const int ppp = 2 * g.pos_per_cta;  // positions per 128-row tile
  const bool folded = g.pack_g == g.group;
  t.q_off = 0, t.k_off = 0, t.kvh = 0, t.kt = 0, t.hu = 0, t.tp = 0, t.n_stages = 0;
  t.u_lo = 0, t.u_hi = 1, t.r_lo = 0, t.r_hi = 0, t.kv_tile = 0, t.carry_in = 0, t.carry_out = 0;
  if (idx < gl.n_kv_pairs) {
    t.mode = idx & 1;
    int i2 = idx >> 1;
    if (g.cu_q == nullptr) {
      t.kt = i2 % p.key_tiles;  // heaviest key tile of a sequence first under a causal mask
      i2 /= p.key_tiles;
      t.b = p.c_b0 + i2 % p.c_nb;
      t.kvh = gl.kv0 + i2 / p.c_nb;
      t.sq = g.seqlen_q, t.sk = g.seqlen_k;
      t.n_row_tiles = g.row_tiles;
      t.tile_base = t.b * g.row_tiles;
      t.kv_tile = t.b * p.key_tiles + t.kt;
    } else {
      t.kvh = gl.kv0 + i2 / p.key_tiles;
      const int r = i2 % p.key_tiles;
      int acc_k = 0, acc_r = 0;
      t.b = -1;
      for (int i = 0; i < g.batch; ++i) {
        const int k0 = g.cu_k[i], k1 = g.cu_k[i + 1], q0 = g.cu_q[i], q1 = g.cu_q[i + 1];
        const int nkt = (k1 - k0 + 255) / 256, nrt = (q1 - q0 + ppp - 1) / ppp;
        if (r < acc_k + nkt) {
          t.b = i, t.kt = r - acc_k, t.sq = q1 - q0, t.sk = k1 - k0, t.q_off = q0, t.k_off = k0, t.n_row_tiles = nrt;
          break;
        }
        acc_k += nkt;
        acc_r += nrt;
      }
      if (t.b < 0) return false;
      t.tile_base = acc_r;
      t.kv_tile = acc_k + t.kt;
      if (t.sk + 64 > p.ws_pitch) return false;  // reported by the tile kernel (ST_BAD_SEQLEN)
    }
    if (t.kvh >= gl.kv1) return false;
    int t_min = 0;
    if (g.causal) {  // first row tile that can see this key tile (bottom-right aligned)
      const int x = t.kt * 256 - (t.sk - t.sq);
      t_min = x > 0 ? x / ppp : 0;
    }
    const int units = folded ? 1 : g.group;
    if (!folded) {
      t.u_lo = max(0, p.c_hu0 - t.kvh * g.group);
      t.u_hi = min(g.group, p.c_hu1 - t.kvh * g.group);
    }
    int lo, hi;
    chunk_tile_range(p, t.tile_base, lo, hi);
    t.r_lo = max(t_min, lo);
    t.r_hi = min(t.n_row_tiles, hi);
    const int rows = max(t.r_hi - t.r_lo, 0), nu = max(t.u_hi - t.u_lo, 0);
    t.n_stages = nu * rows * 2;  // 64-row chunks
    if (t.n_row_tiles - t_min > 0) {
      // the tile's whole sum is (query heads ascending) x (row tiles descending); this chunk holds a box of it
      t.carry_in = (t.u_lo > 0) || (max(t_min, hi) < t.n_row_tiles);
      t.carry_out = (t.u_hi < units) || (t_min < min(lo, t.n_row_tiles));
      if (t.n_stages == 0) return false;  // nothing of it in this chunk: leave its accumulator alone
    } else {
      // no query row sees these keys: zeros, written once, by the chunk that holds the sequence's last tile pair
      const int top = min(t.tile_base + ((max(t.n_row_tiles, 1) - 1) & ~1), p.g_end - 1);
      if (t.u_lo > 0 || top < p.c_g0 || top >= p.c_g1) return false;
    }
  } else {
    t.mode = grad::kModeDQ;
    int i2 = idx - gl.n_kv_pairs;
    if (i2 >= gl.n_dq_pairs) return false;
    if (g.cu_q == nullptr) {
      const int tl = i2 % p.c_ntp;
      i2 /= p.c_ntp;
      t.b = p.c_b0 + i2 % p.c_nb;
      t.hu = p.c_hu0 + i2 / p.c_nb;
      t.tp = p.c_tp0 + (g.causal ? p.c_ntp - 1 - tl : tl);  // heaviest first
      t.sq = g.seqlen_q, t.sk = g.seqlen_k;
      t.n_row_tiles = g.row_tiles;
      t.tile_base = t.b * g.row_tiles;
    } else {
      t.hu = p.c_hu0 + i2 / gl.dq_pairs_per_unit;
      const int r = i2 % gl.dq_pairs_per_unit;
      int acc_p = 0, acc_r = 0;
      t.b = -1;
      for (int i = 0; i < g.batch; ++i) {
        const int q0 = g.cu_q[i], q1 = g.cu_q[i + 1];
        const int nrt = (q1 - q0 + ppp - 1) / ppp, np = (nrt + 1) / 2;
        if (r < acc_p + np) {
          t.b = i, t.tp = r - acc_p, t.sq = q1 - q0, t.q_off = q0, t.n_row_tiles = nrt;
          t.k_off = g.cu_k[i];
          t.sk = g.cu_k[i + 1] - t.k_off;
          if (g.causal) t.tp = np - 1 - t.tp;
          break;
        }
        acc_p += np;
        acc_r += nrt;
      }
      if (t.b < 0) return false;
      t.tile_base = acc_r;
      if (t.sk + 64 > p.ws_pitch) return false;
    }
    if (t.hu >= p.c_hu1 || !chunk_has_tile(p, t.tile_base, 2 * t.tp)) return false;
    t.kvh = folded ? t.hu : t.hu / g.group;
    // key extent written for this tile pair = that of its last tile, in 256-key blocks
    const int t_last = min(2 * t.tp + 1, t.n_row_tiles - 1);
    int kv_hi = t.sk;
    if (g.causal) kv_hi = min(kv_hi, min((t_last + 1) * ppp, t.sq) + t.sk - t.sq);
    t.n_stages = kv_hi > 0 ? (kv_hi + 63) / 64 : 0;  // 64-key chunks; dS is zero beyond kv_hi
  }
  return true;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(grad::kThreads, 1)
splitd_bwd_grad_kernel(const __grid_constant__ CUtensorMap tm_ws, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const BwdParams p, const GradLaunch gl) {
  using namespace grad;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  uint8_t* smem = smem_raw;
  if (smem_base & 1023u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_SMEM_ALIGN);
    return;
  }
  const uint32_t sRing = smem_base, ctrl = smem_base + kOffCtrl;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffCtrl + kAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kOffCtrl + kTmemPtr);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const TileGeom& g = p.g;
  const int ppp = 2 * g.pos_per_cta;  // positions per 128-row tile
  const bool folded = g.pack_g == g.group;
  // cycle counters of one pair (debug[8..15]): where the MMA issuer and one epilogue warp wait (-DSPLITD_PROFILE)
  const bool prof = kProfile && p.debug != nullptr && pair_id == (n_pairs >> 1) && rank == 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(ctrl + kBarFull + 8 * s, 1);
      mbar_init(ctrl + kBarEmpty + 8 * s, 1);
    }
    mbar_init(ctrl + kBarAccDone, 1);
    mbar_init(ctrl + kBarAccFree, 16);  // 8 epilogue warps x 2 CTAs
    tq_init(ctrl + kTileQ, kConsumers);
    fence_mbar_init();
    prefetch_tmap(&tm_ws);
  }
  if (warp == 1) {
    tmem_alloc<2>(ctrl + kTmemPtr, 512);
    tmem_relinquish<2>();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t leader_acc_free = mapa_u32(ctrl + kBarAccFree, 0);
  const TileQueue tq = tq_make(ctrl + kTileQ);
  const int total_tiles = gl.n_kv_pairs + gl.n_dq_pairs;
  GradTile t;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    // The whole warp runs the loop, one elected lane issues the copies (the warp-uniform form spends about
    // half the cycles per stage of a single lane under a divergent branch).
    {
      bool ok = true;
      uint32_t it = 0;
      const uint32_t leader_full0 = mapa_u32(ctrl + kBarFull, 0);
      auto acquire = [&](uint32_t& st, uint32_t& bar, uint32_t& stage) {
        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
        ok = mbar_wait(ctrl + kBarEmpty + 8 * s, ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_LOAD);
        ok = __all_sync(0xffffffffu, ok);
        bar = leader_full0 + 8 * s;
        st = sRing + s * kStageBytes;
        stage = s;
        ++it;
      };
      for (int n = 0; ok; ++n) {
        const int idx = tq_fetch(tq, n, true, abort_flag, p.status);
        if (idx < 0 || idx >= total_tiles) break;
        if (!grad_decode(p, gl, idx, t) || t.n_stages == 0) continue;
        if (t.mode != kModeDQ) {
          const CUtensorMap* tm_b = t.mode == kModeDK ? &tm_q : &tm_do;
          const int qb = g.cu_q ? 0 : t.b;
          const int key0 = t.kt * 256 + rank * 128;
          for (int u = t.u_lo; u < t.u_hi && ok; ++u) {
            const int h = folded ? t.kvh : t.kvh * g.group + u;
            const int plane = (h - p.c_hu0) * 2 + t.mode;
            // last row tile first: under a causal mask the tiles of one KV head start at different rows, and
            // walking down from the common end keeps the pairs that run side by side on the same Q / dO rows
            for (int rt = t.r_hi - 1; rt >= t.r_lo && ok; --rt) {
              for (int c = 0; c < 2 && ok; ++c) {
                uint32_t st = 0, bar = 0, stage = 0;
                acquire(st, bar, stage);
                if (!ok) break;
                const int ws_row = static_cast<int>(chunk_ws_row(p, t.tile_base, rt)) + c * kRowsPerCta;
                const int pos = t.q_off + rt * ppp + c * g.pos_per_cta;
                if (elect_one()) {
                  if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarFull + 8 * stage, 2 * kStageBytes);
                  tma_load_3d_pair(st, &tm_ws, bar, key0, ws_row, plane);
                  tma_load_3d_pair(st + 8192, &tm_ws, bar, key0 + 64, ws_row, plane);
#pragma unroll
                  for (int m = 0; m < 2; ++m) {
                    const int d0 = m * 256 + rank * 128;
                    tma_load_5d_pair(st + 16384 + m * 16384, tm_b, bar, d0, 0, pos, h, qb);
                    tma_load_5d_pair(st + 16384 + m * 16384 + 8192, tm_b, bar, d0 + 64, 0, pos, h, qb);
                  }
                }
                __syncwarp();
              }
            }
          }
        } else {
          const int kb = g.cu_k ? 0 : t.b;
          const int my_tile_ld = min(2 * t.tp + rank, t.n_row_tiles - 1);  // clamped when the last pair has one tile
          const int ws_row = static_cast<int>(chunk_ws_row(p, t.tile_base, my_tile_ld));
          const int plane = (t.hu - p.c_hu0) * 2 + 1;
          for (int c = 0; c < t.n_stages && ok; ++c) {
            uint32_t st = 0, bar = 0, stage = 0;
            acquire(st, bar, stage);
            if (!ok) break;
            if (elect_one()) {
              if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarFull + 8 * stage, 2 * kStageBytes);
              tma_load_3d_pair(st, &tm_ws, bar, c * 64, ws_row, plane);
              tma_load_3d_pair(st + 8192, &tm_ws, bar, c * 64, ws_row + 64, plane);
#pragma unroll
              for (int m = 0; m < 2; ++m) {
                const int d0 = m * 256 + rank * 128;
                tma_load_4d_pair(st + 16384 + m * 16384, &tm_k, bar, d0, t.k_off + c * 64, t.kvh, kb);
                tma_load_4d_pair(st + 16384 + m * 16384 + 8192, &tm_k, bar, d0 + 64, t.k_off + c * 64, t.kvh, kb);
              }
            }
            __syncwarp();
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    // The whole warp runs the loop, one elected lane issues (warp-uniform control flow keeps the cost of
    // waits, descriptor adds and commits well below the 128 cycles one of these MMAs runs for).
    if (rank == 0) {
      bool ok = true;
      uint32_t it = 0;
      int tiles = 0;
      long long t_full = 0, t_free = 0;
      const long long t_begin = prof ? clock64() : 0;
      for (int n = 0; ok; ++n) {
        const int idx = tq_fetch(tq, n, true, abort_flag, p.status);
        if (idx < 0 || idx >= total_tiles) break;
        if (!grad_decode(p, gl, idx, t) || t.n_stages == 0) continue;
        const bool kv = t.mode != kModeDQ;
        const uint32_t idesc = make_idesc(true, kv, true, 256, 256);  // fp16 x fp16 -> fp32
        const uint32_t a_step = kv ? (2048u >> 4) : (32u >> 4);  // 16 contraction elements further
        const uint32_t a_lbo = kv ? 8192u : 16u;
        // The accumulator must be free: drained by the previous tile's epilogue, and (carry_mode) preloaded with
        // what the earlier chunks summed, which the epilogue warps signal once per tile, the first included.
        if (p.carry_mode || tiles > 0) {
          const long long t0 = prof ? clock64() : 0;
          const uint32_t ph = p.carry_mode ? (tiles & 1) : ((tiles - 1) & 1);
          ok = mbar_wait<true>(ctrl + kBarAccFree, ph, abort_flag, p.status, ST_TIMEOUT_MMA);
          ok = __all_sync(0xffffffffu, ok);
          if (prof) t_free += clock64() - t0;
          if (ok) tc_fence_after_sync();
        }
        const uint32_t acc0 = t.carry_in ? 1u : 0u;
        for (int c = 0; c < t.n_stages && ok; ++c) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          const long long t0 = prof ? clock64() : 0;
          ok = mbar_wait(ctrl + kBarFull + 8 * s, ph, abort_flag, p.status, ST_TIMEOUT_MMA);
          ok = __all_sync(0xffffffffu, ok);
          if (prof) t_full += clock64() - t0;
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t st = sRing + s * kStageBytes;
          const uint32_t a0 = desc_lo(st, a_lbo), b0 = desc_lo(st + 16384, 8192);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
#pragma unroll
              for (int m = 0; m < 2; ++m)
                umma_ss<2>(tmem_base + m * 256, desc_join(a0 + k * a_step),
                           desc_join(b0 + ((m * 16384 + k * 2048) >> 4)), idesc, (c | k) | acc0);
            }
            umma_commit_pair(ctrl + kBarEmpty + 8 * s, 3);
            if (c == t.n_stages - 1) umma_commit_pair(ctrl + kBarAccDone, 3);
          }
          __syncwarp();
          ++it;
        }
        ++tiles;
      }
      if (prof && lane == 0) {
        p.debug[8] = static_cast<float>(clock64() - t_begin);
        p.debug[9] = static_cast<float>(t_full);
        p.debug[10] = static_cast<float>(t_free);
        p.debug[11] = static_cast<float>(it);
        p.debug[12] = static_cast<float>(tiles);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ tile scheduler (leader CTA)
    if (rank == 0 && lane == 0)
      tq_schedule(ctrl + kTileQ, p.tile_counters + kCounterGrad, p.tile_counters + kCounterGradDone, pair_id, n_pairs,
                  total_tiles, abort_flag, p.status);
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue: TMEM -> bf16 -> global
    // 8 warps: warp & 3 selects the 32 TMEM lanes (output rows), (warp - 4) / 4 the 256-column half.
    const int q = warp & 3, half = (warp - 4) >> 2;
    const int Lr = q * 32 + (lane & ~3);      // after the transpose it stores rows Lr .. Lr + 3
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + half * 256;
    bool ok = true;
    int tiles = 0;
    long long t_done = 0, t_drain = 0;
    const long long t_begin = prof ? clock64() : 0;
    for (int n = 0; ok; ++n) {
      const int idx = tq_fetch(tq, n, true, abort_flag, p.status);
      if (idx < 0 || idx >= total_tiles) break;
      if (!grad_decode(p, gl, idx, t)) continue;
      const bool live = t.n_stages > 0;
      // this thread's 32-column blocks of the travelling accumulator: [column block][row = TMEM lane][32 floats]
      float* cslot = nullptr;
      if (p.carry_mode && live && t.mode != kModeDQ)
        cslot = carry_slot(p, t.kv_tile, t.mode, rank) + static_cast<int64_t>(half * 8) * (128 * 32) + (q * 32 + lane) * 32;
      if (p.carry_mode && live) {
        if (t.carry_in) {  // the sum of the earlier chunks goes back into the accumulator
#pragma unroll 1
          for (int cb = 0; cb < 8; ++cb) {
            uint32_t a[32];
            const uint4* src = reinterpret_cast<const uint4*>(cslot + static_cast<int64_t>(cb) * (128 * 32));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint4 w = src[i];
              a[4 * i] = w.x, a[4 * i + 1] = w.y, a[4 * i + 2] = w.z, a[4 * i + 3] = w.w;
            }
            tmem_st32(lane_addr + cb * 32, a);
          }
          tmem_st_wait();
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(leader_acc_free);  // cluster-scope release: the peer's TMEM writes
      }
      const long long t0 = prof ? clock64() : 0;
      if (live) {
        ok = mbar_wait(ctrl + kBarAccDone, tiles & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
      }
      const long long t1 = prof ? clock64() : 0;
      t_done += t1 - t0;
      if (live && t.carry_out) {
        // not the last chunk of this tile: the raw fp32 accumulator travels on
#pragma unroll 1
        for (int cb = 0; cb < 8; ++cb) {
          uint32_t a[32];
          tmem_ld32(lane_addr + cb * 32, a);
          tmem_ld_wait();
          uint4* dst = reinterpret_cast<uint4*>(cslot + static_cast<int64_t>(cb) * (128 * 32));
#pragma unroll
          for (int i = 0; i < 8; ++i) dst[i] = make_uint4(a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
        }
        tc_fence_before_sync();  // (carry_mode: the next tile's arrival above follows in program order)
        ++tiles;
        continue;
      }
      // destination rows of the four rows this thread stores (chunk lane & 3 of each), and the power of two
      // that takes the fp16 scale of P / dS out again
      uint16_t* drow[4];
      bool store[4];
      float unscale;
      if (t.mode != kModeDQ) {
        uint16_t* base = reinterpret_cast<uint16_t*>(t.mode == kModeDK ? p.dk : p.dv);
        const int64_t sb = t.mode == kModeDK ? p.dk_stride_b : p.dv_stride_b;
        const int64_t ss = t.mode == kModeDK ? p.dk_stride_s : p.dv_stride_s;
        const int64_t sh = t.mode == kModeDK ? p.dk_stride_h : p.dv_stride_h;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int key = t.kt * 256 + rank * 128 + Lr + j;
          drow[j] = base + (g.cu_q ? 0 : t.b * sb) + static_cast<int64_t>(t.k_off + key) * ss + t.kvh * sh;
          store[j] = key < t.sk;
        }
      } else {
        const int my_tile = 2 * t.tp + rank;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = Lr + j;
          const int pos = my_tile * ppp + row / g.pack_g;
          const int head = g.pack_g > 1 ? t.hu * g.pack_g + row % g.pack_g : t.hu;
          drow[j] = reinterpret_cast<uint16_t*>(p.dq) + (g.cu_q ? 0 : t.b * p.dq_stride_b) +
                    static_cast<int64_t>(t.q_off + pos) * p.dq_stride_s + static_cast<int64_t>(head) * p.dq_stride_h;
          store[j] = my_tile < t.n_row_tiles && pos < t.sq;
        }
      }
      {
        const uint32_t* st = p.stats + static_cast<int64_t>(t.b * g.heads_kv + t.kvh) * kStatWords;
        unscale = pow2i(t.mode == kModeDV ? -(kPShift + do_exponent(st)) : -ds_exponent(st, p.scale));
      }
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {  // 64 accumulator columns per step
        uint32_t x[32];
        if (live) {
          uint32_t a[32], b[32];
          tmem_ld32(lane_addr + c * 64, a);
          tmem_ld32(lane_addr + c * 64 + 32, b);
          tmem_ld_wait();
          if (c == 3) {  // accumulator read: the next tile's first MMA may overwrite it
            tc_fence_before_sync();
            if (!p.carry_mode) {
              __syncwarp();
              if (lane == 0) mbar_arrive_remote(leader_acc_free);
            }
            if (prof) t_drain += clock64() - t1;
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            x[i] = pack2<false>(__uint_as_float(a[2 * i]) * unscale, __uint_as_float(a[2 * i + 1]) * unscale);
            x[16 + i] = pack2<false>(__uint_as_float(b[2 * i]) * unscale, __uint_as_float(b[2 * i + 1]) * unscale);
          }
          // 64 columns x 2 bytes = 4 chunks of 32 bytes of this thread's row; after the transpose the thread
          // holds chunk (lane & 3) of rows Lr .. Lr + 3, so each 256-bit store instruction of the warp writes
          // whole 128-byte lines
          transpose_chunks32_4x4(x, lane);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) x[i] = 0u;
        }
        const int col = half * 256 + c * 64 + (lane & 3) * 16;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (store[j]) st_global_32b(drow[j] + col, &x[8 * j]);
      }
      if (live) ++tiles;
    }
    if (prof && warp == 4 && lane == 0) {
      p.debug[13] = static_cast<float>(clock64() - t_begin);
      p.debug[14] = static_cast<float>(t_done);
      p.debug[15] = static_cast<float>(t_drain);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc<2>(tmem_base, 512);
  }
}

// modes: bit 0 = dK and dV, bit 1 = dQ
int launch_bwd_grad(const splitd_params* p, const BwdPlan& pl, int chunk, cudaStream_t stream, int modes) {
  BwdParams bp;
  if (int e = fill_bwd_params(p, bp, &pl)) return e;
  plan_chunk(pl, chunk, p, bp);
  const TileGeom& g = bp.g;
  const int nhu = bp.c_hu1 - bp.c_hu0;
  CUtensorMap tm_ws, tm_do, tm_q, tm_k;
  {
    const uint64_t dims[3] = {(uint64_t)bp.ws_pitch, (uint64_t)bp.ws_rows, (uint64_t)(2 * nhu)};
    const int64_t strides[3] = {1, bp.ws_pitch, bp.ws_rows * bp.ws_pitch};
    const uint32_t box[3] = {64, 64, 1};
    if (int e = make_tmap(&tm_ws, bp.ws, 3, dims, strides, box, "workspace")) return e;
  }
  const bool varlen = p->cu_seqlens_q != nullptr;
  {  // the fp16 copies are contiguous (B,S,H,512) / (T,H,512)
    const int64_t sq = varlen ? p->total_q : p->seqlen_q, sk = varlen ? p->total_k : p->seqlen_k;
    const int64_t qs[3] = {sq * p->heads_q * kHeadDim, static_cast<int64_t>(p->heads_q) * kHeadDim, kHeadDim};
    const int64_t ks[3] = {sk * p->heads_kv * kHeadDim, static_cast<int64_t>(p->heads_kv) * kHeadDim, kHeadDim};
    if (int e = make_q_tmap(&tm_do, bp.do_h, p, g, qs, g.pos_per_cta, "dout (fp16 copy)")) return e;
    if (int e = make_q_tmap(&tm_q, bp.q_h, p, g, qs, g.pos_per_cta, "q (fp16 copy)")) return e;
    if (int e = make_kv_tmap(&tm_k, bp.k_h, p, ks, 64, "k (fp16 copy)")) return e;
  }
  const bool folded = g.pack_g == g.group;
  GradLaunch gl;
  gl.kv0 = folded ? bp.c_hu0 : bp.c_hu0 / g.group;
  gl.kv1 = folded ? bp.c_hu1 : (bp.c_hu1 - 1) / g.group + 1;
  gl.dq_pairs_per_unit = varlen ? (g.row_tiles + g.batch + 1) / 2 : (g.row_tiles + 1) / 2;
  long long kv = 2ll * bp.key_tiles * (gl.kv1 - gl.kv0) * (varlen ? 1 : bp.c_nb);
  long long dq = varlen ? static_cast<long long>(gl.dq_pairs_per_unit) * nhu : static_cast<long long>(bp.c_ntp) * bp.c_nb * nhu;
  if (!(modes & 1)) kv = 0;
  if (!(modes & 2)) dq = 0;
  if ((modes & 3) != 3 && pl.n_chunks > 1)
    return fail(SPLITD_ERR_WORKSPACE, "dq and dk/dv as separate steps need the whole problem in one chunk");
  const long long pairs = kv + dq;
  if (pairs <= 0 || pairs > (1ll << 30)) return fail(SPLITD_ERR_INVALID_ARGUMENT, "gradient GEMM grid out of range");
  gl.n_kv_pairs = static_cast<int>(kv);
  gl.n_dq_pairs = static_cast<int>(dq);
  // persistent: as many CTA pairs as the device keeps resident at once
  static std::atomic<int> cache[64];
  const int resident = resident_cluster_pairs(splitd_bwd_grad_kernel, grad::kThreads, grad::kSmemBytes, cache);
  if (resident <= 0) return fail(SPLITD_ERR_CUDA, "cudaFuncSetAttribute(gradient GEMM kernel) failed");
  const long long grid_pairs = pairs < resident ? pairs : resident;
  splitd_bwd_grad_kernel<<<dim3(static_cast<unsigned>(2 * grid_pairs)), dim3(grad::kThreads), grad::kSmemBytes,
                           stream>>>(tm_ws, tm_do, tm_q, tm_k, bp, gl);
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "gradient GEMM launch failed: %s", cudaGetErrorString(ce));
  return 0;
}

int launch_bwd_chunk(const splitd_params* p, const BwdPlan& pl, int chunk, int stages, cudaStream_t stream) {
  if (stages & 1)
    if (int e = launch_bwd_pds(p, pl, chunk, stream)) return e;
  const int modes = ((stages & 2) ? 1 : 0) | ((stages & 4) ? 2 : 0);
  if (modes) return launch_bwd_grad(p, pl, chunk, stream, modes);
  return 0;
}

}  // namespace sd
