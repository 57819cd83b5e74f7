// Backward step 2a: the P and dS tiles.  S = Q K^T, dP = dO V^T on the tensor cores, then
//     P = exp2(S*scale*log2e - lse_log2),   dS = P * (dP - dpsum) * scale
// (src/fmha_dq_sm90_d512.py:1040-1090 / src/fmha_dkdv_sm90_d512.py:1060-1130 of the reference) are written
// as bf16 to the workspace, rows in packed order, so that dQ, dK and dV are three plain GEMMs over them
// (bwd_grad_kernel.cu) and nothing is recomputed. The reference recomputes S and dP in each of four
// D passes of both of its backward kernels (3.8x the useful FLOPs).
//
// CTA pair, cta_group::2 UMMAs with M = 128 (64 packed rows per CTA), N = 256 keys per step. No accumulator
// lives across steps, so TMEM holds two (S, dP) buffer pairs of 128 + 128 columns: the tensor pipe fills one
// pair while eight element-wise warps drain the other.
// What bounds this kernel is the operand stream: a load takes ~1700 cycles from issue to landing, so the
// bytes per cycle it delivers are (ring bytes in flight) / 1700, and with Q and dO both resident (128 KB) only
// 96 KB of ring were left for 256 KB of K/V per step. Hence only dO (64 x 512) stays resident; the Q tile is
// re-streamed with the K rows (an 8 KB Q block rides in every K stage, +25 % L2 traffic), which buys rings of
// 4 x 24 KB (K rows + Q block) for the QK^T issuer and 4 x 16 KB (V rows) for the dO V^T issuer.
// Persistent pairs: one pair per SM pair draws tiles (heaviest first under a causal mask) from a work counter
// (tile_queue.cuh); QK^T of the next tile starts while the last stores of the previous one are still going
// out, and only the dO reload (64 KB) waits for the previous tile's last dO V^T MMA.
// A tile pair (even tile, odd tile) always writes the same number of 256-key blocks (the odd tile's), so
// the dQ GEMM can run both tiles of a pair over one key range; the surplus block of the even tile is
// fully masked and therefore zero.
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"
#include "tile_queue.cuh"

namespace sd {

namespace pds {
constexpr int kStepKeys = 256;
constexpr int kStages = 4;            // per ring; one ring for K rows (+ Q block), one for V rows
constexpr int kBoxBytes = 16384;      // one K / V TMA box: this CTA's 128 keys x 64 of the 512 D columns
constexpr int kQBoxBytes = 8192;      // the tile's 64 rows x the same 64 D columns of Q
constexpr int kStageK = kBoxBytes + kQBoxBytes;
constexpr int kStageV = kBoxBytes;
constexpr int kOffDO = 0;
constexpr int kOffRingK = 65536;
constexpr int kOffRingV = kOffRingK + kStages * kStageK;
constexpr int kOffCtrl = kOffRingV + kStages * kStageV;
constexpr int kBarFullK = 0;
constexpr int kBarEmptyK = kBarFullK + 8 * kStages;
constexpr int kBarFullV = kBarEmptyK + 8 * kStages;
constexpr int kBarEmptyV = kBarFullV + 8 * kStages;
constexpr int kBarSdpFull = kBarEmptyV + 8 * kStages;  // [2], two arrivals each: the S issuer's and the dP issuer's commit
constexpr int kBarSdpFree = kBarSdpFull + 16;          // [2], leader CTA only
constexpr int kBarDoFull = kBarSdpFree + 16;
constexpr int kBarDoFree = kBarDoFull + 8;             // the dO V^T issuer's last MMA of a tile has read dO
constexpr int kTmemPtr = kBarDoFree + 8;
constexpr int kAbort = kTmemPtr + 4;
constexpr int kTileQ = kAbort + 4;                     // TileQueue, kTileQueueBytes
constexpr int kCtrlBytes = 256;
constexpr int kSmemBytes = kOffCtrl + kCtrlBytes;
constexpr int kConsumers = 2 + 2 + 16;  // producers of both CTAs, the two issuers, element-wise warps of both CTAs
static_assert(kSmemBytes <= 232448, "shared memory budget");
static_assert(kTileQ % 8 == 0 && kTileQ + kTileQueueBytes <= kCtrlBytes, "control block overflow");
}  // namespace pds

// Number of 256-key steps of a tile: the key extent is that of the odd tile of the tile's pair (see header).
__device__ __forceinline__ int pds_tile_steps(const TileGeom& g, const TileCoord& tc) {
  int kv_hi = tc.sk;
  if (g.causal) {
    const int ppp = 2 * g.pos_per_cta;
    const int n_tiles = (tc.sq + ppp - 1) / ppp;
    const int t_last = min(tc.rt | 1, n_tiles - 1);
    const int last_pos = min((t_last + 1) * ppp, tc.sq) - 1;
    kv_hi = min(kv_hi, last_pos + 1 + tc.sk - tc.sq);
  }
  return kv_hi > 0 ? (kv_hi + pds::kStepKeys - 1) / pds::kStepKeys : 0;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(384, 1)
splitd_bwd_pds_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                      const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const BwdParams p, const int total_tiles) {
  using namespace pds;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  uint8_t* smem = smem_raw;
  if (smem_base & 1023u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_SMEM_ALIGN);
    return;
  }
  const uint32_t sDO = smem_base + kOffDO;
  const uint32_t sRingK = smem_base + kOffRingK, sRingV = smem_base + kOffRingV, ctrl = smem_base + kOffCtrl;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffCtrl + kAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kOffCtrl + kTmemPtr);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const TileGeom& g = p.g;

  // optional cycle counters of one pair (debug[0..5]), summed over its tiles
  const bool prof = p.debug != nullptr && pair_id == (n_pairs >> 1) && rank == 0;
  long long t_a = 0, t_b = 0, t_c = 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(ctrl + kBarDoFull, 1);
    mbar_init(ctrl + kBarDoFree, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(ctrl + kBarFullK + 8 * s, 1);
      mbar_init(ctrl + kBarEmptyK + 8 * s, 1);
      mbar_init(ctrl + kBarFullV + 8 * s, 1);
      mbar_init(ctrl + kBarEmptyV + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(ctrl + kBarSdpFull + 8 * b, 2);
      mbar_init(ctrl + kBarSdpFree + 8 * b, 16);  // 8 element-wise warps x 2 CTAs
    }
    tq_init(ctrl + kTileQ, kConsumers);
    fence_mbar_init();
    prefetch_tmap(&tm_q);
    prefetch_tmap(&tm_do);
    prefetch_tmap(&tm_k);
    prefetch_tmap(&tm_v);
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
  const TileQueue tq = tq_make(ctrl + kTileQ);
  TileCoord tc;

  if (warp == 0) {
    // TMA producer: the whole warp runs the loop, one elected lane issues (same reason as for the MMA issuers
    // below: the warp-uniform form spends about half the cycles per stage, and a busy producer is latency
    // added to every freed ring slot).
    const uint32_t leader_do_full = mapa_u32(ctrl + kBarDoFull, 0);
    const uint32_t leader_full_k = mapa_u32(ctrl + kBarFullK, 0), leader_full_v = mapa_u32(ctrl + kBarFullV, 0);
    uint32_t it = 0;     // ring stage pairs issued so far (all tiles)
    uint32_t tiles = 0;  // tiles with work so far
    bool ok = true;
    for (int n = 0; ok; ++n) {
      const int idx = tq_fetch(tq, n, true, abort_flag, p.status);
      if (idx < 0 || idx >= total_tiles) break;
      if (!decode_tile(g, idx, tc)) continue;
      const int n_steps = pds_tile_steps(g, tc);
      if (n_steps == 0) continue;
      const int qpos = tc.q_off + tc.p0 + static_cast<int>(rank) * g.pos_per_cta;
      const int qb = g.cu_q ? 0 : tc.b;
      const int kb = g.cu_k ? 0 : tc.b;
      bool do_pending = true;
      for (int j = 0; j < n_steps && ok; ++j) {
        const int key0 = tc.k_off + j * kStepKeys + static_cast<int>(rank) * 128;
        for (int c = 0; c < 8 && ok; ++c) {  // K and V boxes alternate so that both issuers are fed evenly
          if (do_pending && c == kStages) {
            // dO of this tile, once the ring holds the tile's first stages: the buffer is free when the previous
            // tile's last dO V^T MMA has completed (the first stages above do not depend on it, so QK^T of the
            // new tile already runs while dO is on its way)
            if (tiles > 0) {
              ok = mbar_wait(ctrl + kBarDoFree, (tiles - 1) & 1, abort_flag, p.status, ST_TIMEOUT_LOAD);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
            }
            if (elect_one()) {
              if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarDoFull, 2 * 65536);
              for (int d = 0; d < 8; ++d)
                tma_load_5d_pair(sDO + d * 8192, &tm_do, leader_do_full, d * 64, 0, qpos, tc.hu, qb);
            }
            __syncwarp();
            do_pending = false;
          }
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          ok = mbar_wait(ctrl + kBarEmptyK + 8 * s, ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_LOAD);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (elect_one()) {
            if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarFullK + 8 * s, 2 * kStageK);
            tma_load_4d_pair(sRingK + s * kStageK, &tm_k, leader_full_k + 8 * s, c * 64, key0, tc.hkv, kb);
            tma_load_5d_pair(sRingK + s * kStageK + kBoxBytes, &tm_q, leader_full_k + 8 * s, c * 64, 0, qpos, tc.hu, qb);
          }
          __syncwarp();
          ok = mbar_wait(ctrl + kBarEmptyV + 8 * s, ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_LOAD);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (elect_one()) {
            if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarFullV + 8 * s, 2 * kStageV);
            tma_load_4d_pair(sRingV + s * kStageV, &tm_v, leader_full_v + 8 * s, c * 64, key0, tc.hkv, kb);
          }
          __syncwarp();
          ++it;
        }
      }
      ++tiles;
    }
  } else if (warp == 1 || warp == 2) {
    // Two issuing warps: warp 1 issues the S = Q K^T MMAs from the K ring, warp 2 the dP = dO V^T MMAs from
    // the V ring, so each GEMM has its own instruction stream and its own operand prefetch. In each the whole
    // warp runs the loop and one elected lane issues: warp-uniform control flow makes waits, descriptor adds
    // and commits cost ~42 cycles per MMA instead of ~85 for a single lane under a divergent branch (both
    // measured), which is what keeps the 64-cycle MMAs of this shape back to back.
    if (rank == 0) {
      const bool is_s = warp == 1;
      constexpr uint32_t idesc = make_idesc(false, false, false, 128, kStepKeys);
      const uint32_t do_lo = desc_lo(sDO, 16), ring_lo = desc_lo(is_s ? sRingK : sRingV, 16);
      const uint32_t stage16 = (is_s ? kStageK : kStageV) >> 4;
      const uint32_t bar_full = ctrl + (is_s ? kBarFullK : kBarFullV), bar_empty = ctrl + (is_s ? kBarEmptyK : kBarEmptyV);
      const uint32_t d_off = is_s ? 0 : 128;
      const bool prof_t = prof && is_s;
      uint32_t it = 0;     // ring stages consumed (all tiles)
      uint32_t gs = 0;     // steps issued (all tiles): S/dP buffer pair and barrier phases follow it
      uint32_t tiles = 0;  // tiles with work so far
      bool ok = true;
      const long long t_begin = prof_t ? clock64() : 0;
      for (int n = 0; ok; ++n) {
        const int idx = tq_fetch(tq, n, true, abort_flag, p.status);
        if (idx < 0 || idx >= total_tiles) break;
        if (!decode_tile(g, idx, tc)) continue;
        const int n_steps = pds_tile_steps(g, tc);
        if (n_steps == 0) continue;
        if (!is_s) {  // this tile's dO has landed
          ok = mbar_wait(ctrl + kBarDoFull, tiles & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
        }
        for (int j = 0; j < n_steps && ok; ++j, ++gs) {
          const uint32_t b = gs & 1;
          if (gs >= 2) {  // buffer pair b must have been drained
            const long long t0 = prof_t ? clock64() : 0;
            ok = mbar_wait<true>(ctrl + kBarSdpFree + 8 * b, ((gs >> 1) - 1) & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
            ok = __all_sync(0xffffffffu, ok);
            if (prof_t) t_b += clock64() - t0;
            if (!ok) break;
            tc_fence_after_sync();
          }
          const uint32_t d_tmem = tmem_base + b * 256 + d_off;
          const bool last_step = j == n_steps - 1;
#pragma unroll 1
          for (int c = 0; c < 8 && ok; ++c) {
            const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
            const long long t0 = prof_t ? clock64() : 0;
            ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status, ST_TIMEOUT_MMA);
            ok = __all_sync(0xffffffffu, ok);
            if (prof_t) t_a += clock64() - t0;
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t b0 = ring_lo + s * stage16;
            // A: the Q block that came with this K stage / the resident dO block of the same 64 D columns
            const uint32_t a0 = is_s ? b0 + (kBoxBytes >> 4) : do_lo + c * (8192 >> 4);
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                umma_ss<2>(d_tmem, desc_join(a0 + ((k * 32) >> 4)), desc_join(b0 + ((k * 32) >> 4)), idesc, (c | k) != 0);
              umma_commit_pair(bar_empty + 8 * s, 3);
              if (c == 7) {
                umma_commit_pair(ctrl + kBarSdpFull + 8 * b, 3);
                if (!is_s && last_step) umma_commit_pair(ctrl + kBarDoFree, 3);  // dO may be overwritten
              }
            }
            __syncwarp();
            ++it;
          }
        }
        ++tiles;
      }
      if (prof_t && lane == 0) {
        p.debug[0] = static_cast<float>(t_a);
        p.debug[1] = static_cast<float>(t_b);
        p.debug[2] = static_cast<float>(clock64() - t_begin);
        p.debug[3] = static_cast<float>(gs);
      }
    }
  } else if (warp == 3) {
    // tile scheduler (leader CTA)
    if (rank == 0 && lane == 0)
      tq_schedule(ctrl + kTileQ, p.tile_counters + kCounterPds, pair_id, n_pairs, total_tiles, abort_flag, p.status);
  } else if (warp >= 4) {
    const int q = warp & 3, wg = (warp - 4) >> 2;
    const int L = q * 32 + lane;
    const int row = L & 63, half = L >> 6;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int64_t plane = p.ws_rows * p.ws_pitch;
    const uint32_t leader_free0 = mapa_u32(ctrl + kBarSdpFree, 0);
    bool ok = true;
    uint32_t gs = 0;  // steps seen (all tiles), same counter as the issuers'
    uint32_t s[64], d[32];  // S / P of this thread's 64 keys; one 32-column slice of dP
    const long long t_begin = prof ? clock64() : 0;
    for (int n = 0; ok; ++n) {
      const int idx = tq_fetch(tq, n, true, abort_flag, p.status);
      if (idx < 0 || idx >= total_tiles) break;
      if (!decode_tile(g, idx, tc)) continue;
      const int n_steps = pds_tile_steps(g, tc);
      if (n_steps == 0) continue;
      const int pos = tc.p0 + static_cast<int>(rank) * g.pos_per_cta + row / g.pack_g;
      const int head = (g.pack_g > 1) ? tc.hu * g.pack_g + row % g.pack_g : tc.hu;
      const bool row_ok = pos < tc.sq;
      int limit = tc.sk - 1;
      if (g.causal) limit = min(limit, pos + tc.sk - tc.sq);
      if (!row_ok) limit = -1;
      float lse2 = 0.f, delta = 0.f;
      if (row_ok) {
        const int64_t ridx = g.cu_q ? static_cast<int64_t>(head) * p.total_q + tc.q_off + pos
                                    : (static_cast<int64_t>(tc.b) * g.heads_q + head) * tc.sq + pos;
        lse2 = p.lse_log2[ridx];
        delta = p.dpsum[ridx];
      }
      const float nds = -delta * p.scale;
      uint16_t* ws_p = p.ws + (static_cast<int64_t>(tc.hu) * 2) * plane +
                       (static_cast<int64_t>(tc.tile_global) * kRowsPerPair + rank * kRowsPerCta + row) * p.ws_pitch;

      for (int j = 0; j < n_steps && ok; ++j, ++gs) {
        const uint32_t b = gs & 1;
        const long long t0 = prof ? clock64() : 0;
        ok = mbar_wait(ctrl + kBarSdpFull + 8 * b, (gs >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
        if (prof) t_c += clock64() - t0;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t s_addr = lane_addr + b * 256 + wg * 64;
        const int key0 = j * kStepKeys + half * 128 + wg * 64;
        const int cl = limit - key0;
        tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
        tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
        tmem_ld_wait();
        // P (fp32, kept in s[]); masked entries are forced to zero (warp-uniform fast path without masks)
        const bool full = __all_sync(0xffffffffu, cl >= 63);
        if (full) {
#pragma unroll
          for (int i = 0; i < 64; ++i) s[i] = __float_as_uint(ex2(fmaf(__uint_as_float(s[i]), p.scale_log2, -lse2)));
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const float pv = ex2(fmaf(__uint_as_float(s[i]), p.scale_log2, -lse2));
            s[i] = __float_as_uint(i > cl ? 0.f : pv);
          }
        }
        uint32_t dk[32];
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          tmem_ld32(s_addr + 128 + c2 * 32, d);
          tmem_ld_wait();
          if (c2 == 1) {  // both buffers of this step have been read: hand them back to the tensor pipe
            tc_fence_before_sync();
            __syncwarp();
            // cluster-scope release on purpose: its memory barrier paces these warps (their global stores
            // compete with the K/V stream that bounds this kernel), which measures ~4-7 % faster than the
            // cheaper CTA-scope arrive used elsewhere
            if (lane == 0) mbar_arrive_cluster(leader_free0 + 8 * b);
          }
          // dS = P * (dP - delta) * scale = P * fma(dP, scale, -delta*scale); P is already 0 where masked,
          // the select only guards against non-finite dP of rows/keys outside the sequence
          if (full) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float a = __uint_as_float(s[c2 * 32 + i]) * fmaf(__uint_as_float(d[i]), p.scale, nds);
              const float bb = __uint_as_float(s[c2 * 32 + i + 1]) * fmaf(__uint_as_float(d[i + 1]), p.scale, nds);
              dk[c2 * 16 + (i >> 1)] = pack2<false>(a, bb);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = __uint_as_float(s[c2 * 32 + i]), p1 = __uint_as_float(s[c2 * 32 + i + 1]);
              const float a = (c2 * 32 + i > cl) ? 0.f : p0 * fmaf(__uint_as_float(d[i]), p.scale, nds);
              const float bb = (c2 * 32 + i + 1 > cl) ? 0.f : p1 * fmaf(__uint_as_float(d[i + 1]), p.scale, nds);
              dk[c2 * 16 + (i >> 1)] = pack2<false>(a, bb);
            }
          }
        }
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 64; i += 2) pk[i >> 1] = pack2<false>(__uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        // 64 keys x 2 bytes = 4 chunks of 32 bytes per row; transpose inside groups of 4 lanes so that every
        // 256-bit store instruction writes 8 whole 128-byte lines (instead of 32 partial ones)
        transpose_chunks32_4x4(pk, lane);
        transpose_chunks32_4x4(dk, lane);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          // this thread now holds chunk (lane & 3) of row (lane & ~3) + r; its own row is `lane`
          const int64_t row_delta = static_cast<int64_t>((lane & ~3) + r - lane) * p.ws_pitch;
          uint16_t* dst_p = ws_p + row_delta + key0 + (lane & 3) * 16;
          st_global_v8(dst_p, &pk[8 * r]);
          st_global_v8(dst_p + plane, &dk[8 * r]);
        }
      }
    }
    if (prof && warp == 4 && lane == 0) {
      p.debug[4] = static_cast<float>(t_c);
      p.debug[5] = static_cast<float>(clock64() - t_begin);
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

int launch_bwd_pds(const splitd_params* p, cudaStream_t stream) {
  // Default: the two-pass form (bwd_pds2_kernel.cu). SPLITD_PDS_ONE_PASS=1 in the environment selects the
  // one-pass kernel below, which moves 2 bytes per (row, key) less through HBM but streams K/V at twice the
  // bytes per FLOP; it is read once per process.
  static const int one_pass = [] { const char* e = getenv("SPLITD_PDS_ONE_PASS"); return e && e[0] == '1'; }();
  if (!one_pass) return launch_bwd_pds_two_pass(p, stream);
  BwdParams bp;
  if (int e = fill_bwd_params(p, bp)) return e;
  if (int e = check_workspace(p)) return e;
  const TileGeom& g = bp.g;
  CUtensorMap tm_q, tm_do, tm_k, tm_v;
  if (int e = make_q_tmap(&tm_q, p->q, p, g, p->q_strides, g.pos_per_cta, "q")) return e;
  if (int e = make_q_tmap(&tm_do, p->dout, p, g, p->do_strides, g.pos_per_cta, "dout")) return e;
  if (int e = make_kv_tmap(&tm_k, p->k, p, p->k_strides, 128, "k")) return e;
  if (int e = make_kv_tmap(&tm_v, p->v, p, p->v_strides, 128, "v")) return e;
  const bool varlen = p->cu_seqlens_q != nullptr;
  const long long pairs = varlen ? static_cast<long long>(g.row_tiles) * g.head_units
                                 : static_cast<long long>(g.row_tiles) * g.head_units * g.batch;
  if (pairs <= 0 || pairs > (1ll << 30)) return fail(SPLITD_ERR_INVALID_ARGUMENT, "P/dS grid out of range");
  cudaError_t ce =
      cudaFuncSetAttribute(splitd_bwd_pds_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pds::kSmemBytes);
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "cudaFuncSetAttribute(pds): %s", cudaGetErrorString(ce));
  // persistent: as many CTA pairs as the device keeps resident at once; tiles are drawn from a work counter
  static int cache[64] = {};
  const int resident = resident_cluster_pairs(splitd_bwd_pds_kernel, 384, pds::kSmemBytes, cache);
  const long long grid_pairs = pairs < resident ? pairs : resident;
  ce = cudaMemsetAsync(bp.tile_counters + kCounterPds, 0, sizeof(int), stream);
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "cudaMemsetAsync(tile counter): %s", cudaGetErrorString(ce));
  splitd_bwd_pds_kernel<<<dim3(static_cast<unsigned>(2 * grid_pairs)), dim3(384), pds::kSmemBytes, stream>>>(
      tm_q, tm_do, tm_k, tm_v, bp, static_cast<int>(pairs));
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "P/dS launch failed: %s", cudaGetErrorString(ce));
  return 0;
}

}  // namespace sd
