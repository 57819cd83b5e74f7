// Backward step 2a: the P and dS tiles, from two GEMM passes that alternate inside one kernel.
//     pass 0:  S  = Q K^T      ->  P  = exp2(S*scale*log2e - lse_log2)          (written to the workspace)
//     pass 1:  dP = dO V^T     ->  dS = P * (dP - dpsum) * scale                (P read back, dS written)
// (the math of src/fmha_dq_sm90_d512.py:1040-1090 / src/fmha_dkdv_sm90_d512.py:1060-1130 of the reference).
// Both are stored as fp16 with power-of-two scales (bwd_common.cuh): three more significant bits than bf16 at
// the same bytes, which is what keeps dQ and dK within twice the error of a result that is rounded once.
//
// Why two passes: with ONE resident A operand (Q or dO) a CTA can hold 128 rows of it (128 KB), so every MMA
// is a cta_group::2 UMMA with M = 256 (128 rows per CTA, TMEM lane = row), N = 256 keys: 128 cycles per
// MMA for 4 KB of streamed B operand per CTA instead of 64 cycles, i.e. half the K/V bytes per FLOP of a
// kernel that does both GEMMs per key step with 64 rows per CTA (measured 6 % slower on this step).
// Why they alternate: a pair runs pass 0 over a chunk of kChunkSteps key steps and then pass 1 over the same
// chunk, so the P values pass 1 reads (<= 0.5 MB per pair) are still in L2 and HBM sees each tile element twice
// (P out, dS out) like in the one-pass kernel. The resident operand is swapped at every pass switch, block by
// block as the previous pass's last step releases it.
//
// CTA pair = two 128-row tiles (even, odd) of one (batch, head unit); CTA c owns tile 2*tp + c. The pair
// runs over the key range of its odd tile (the later one under a causal mask); blocks that are masked for
// the even tile come out as zeros, which is what the gradient GEMMs expect.
// Shared memory: A resident (128 x 512 bf16 = 128 KB in eight 64-column blocks), B ring 6 x 16 KB. TMEM: two
// 256-column buffers. Persistent pairs drawing tiles from a work counter (tile_queue.cuh); whole-warp issue
// loops with an elected lane (a stage loop run by one lane under a divergent branch costs twice the cycles).
// One launch covers one chunk of the problem (BwdParams::c_*): the head units and row tiles whose planes the
// workspace currently holds.
#include <cstring>

#include "bwd_common.cuh"
#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"
#include "tile_queue.cuh"

namespace sd {

namespace pds2 {
constexpr int kStepKeys = 256;
constexpr int kChunkSteps = 4;       // key steps per pass before the pair switches to the other pass (8, 16: +-2 %)
constexpr int kStages = 6;
constexpr int kStageBytes = 16384;   // this CTA's 128 keys x 64 of the 512 D columns
constexpr int kABlockBytes = 16384;  // the tile's 128 rows x the same 64 D columns
constexpr int kOffA = 0;
constexpr int kOffRing = 8 * kABlockBytes;
constexpr int kOffCtrl = kOffRing + kStages * kStageBytes;
constexpr int kBarFull = 0;
constexpr int kBarEmpty = kBarFull + 8 * kStages;
constexpr int kBarAFull = kBarEmpty + 8 * kStages;  // [8] one per 64-column block of A
constexpr int kBarAFree = kBarAFull + 64;           // [8]
constexpr int kBarOutFull = kBarAFree + 64;         // [2]
constexpr int kBarOutFree = kBarOutFull + 16;       // [2], leader CTA only
constexpr int kTmemPtr = kBarOutFree + 16;
constexpr int kAbort = kTmemPtr + 4;
constexpr int kTileQ = kAbort + 4;
constexpr int kCtrlBytes = 320;
constexpr int kSmemBytes = kOffCtrl + kCtrlBytes;
constexpr int kThreads = 384;
constexpr int kConsumers = 2 + 1 + 16;  // producers of both CTAs, the MMA issuer, element-wise warps of both CTAs
static_assert(kTileQ % 8 == 0 && kTileQ + kTileQueueBytes <= kCtrlBytes, "control block overflow");
static_assert(kSmemBytes <= 232448, "shared memory budget");
}  // namespace pds2

struct PairTile {
  int b, hu, hkv, tp;
  int sq, sk, q_off, k_off;
  int tile_base, n_row_tiles;
  int n_steps;
};

// Tile pair `idx` of the launch (heaviest first under a causal mask). `ppu`: tile pairs per head unit over all
// sequences of the packed layout (an upper bound). Returns false for a slot without a tile of this chunk.
__device__ __forceinline__ bool pds2_decode(const BwdParams& p, int ppu, int idx, PairTile& t) {
  const TileGeom& g = p.g;
  const int ppp = 2 * g.pos_per_cta;  // positions per 128-row tile
  t.q_off = 0, t.k_off = 0;
  if (g.cu_q == nullptr) {
    const int tl = idx % p.c_ntp;
    idx /= p.c_ntp;
    t.b = p.c_b0 + idx % p.c_nb;
    t.hu = p.c_hu0 + idx / p.c_nb;
    t.tp = p.c_tp0 + (g.causal ? p.c_ntp - 1 - tl : tl);
    t.sq = g.seqlen_q, t.sk = g.seqlen_k;
    t.n_row_tiles = g.row_tiles;
    t.tile_base = t.b * g.row_tiles;
  } else {
    t.hu = p.c_hu0 + idx / ppu;
    const int r = idx % ppu;
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
    if (t.sk + 64 > p.ws_pitch) {  // the caller's max_seqlen_k was too small for this sequence: no row to write to
      if (p.status) atomicCAS(p.status, 0, ST_BAD_SEQLEN);
      return false;
    }
  }
  if (t.hu >= p.c_hu1 || !chunk_has_tile(p, t.tile_base, 2 * t.tp)) return false;
  t.hkv = (g.pack_g == g.group) ? t.hu : t.hu / g.group;
  const int t_last = min(2 * t.tp + 1, t.n_row_tiles - 1);
  int kv_hi = t.sk;
  if (g.causal) kv_hi = min(kv_hi, min((t_last + 1) * ppp, t.sq) + t.sk - t.sq);
  t.n_steps = kv_hi > 0 ? (kv_hi + pds2::kStepKeys - 1) / pds2::kStepKeys : 0;
  return true;
}

__device__ __forceinline__ void ld_global_v8_hint(const void* p, uint32_t* w, uint64_t policy) {
  asm volatile("ld.global.L2::cache_hint.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8], %9;"
               : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
               : "l"(p), "l"(policy)
               : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(pds2::kThreads, 1)
splitd_bwd_pds2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const BwdParams p, const int total_tiles, const int ppu) {
  using namespace pds2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  uint8_t* smem = smem_raw;
  if (smem_base & 1023u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_SMEM_ALIGN);
    return;
  }
  const uint32_t sA = smem_base + kOffA, sRing = smem_base + kOffRing, ctrl = smem_base + kOffCtrl;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffCtrl + kAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kOffCtrl + kTmemPtr);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_ctarank());
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const TileGeom& g = p.g;
  const int ppp = 2 * g.pos_per_cta;

  // cycle counters of one pair (debug[0..7]), summed over its tiles; compiled in with -DSPLITD_PROFILE only
  const bool prof = kProfile && p.debug != nullptr && pair_id == (n_pairs >> 1) && rank == 0;
  float* dbg = p.debug;
  long long t_a = 0, t_b = 0, t_c = 0, t_m0 = 0, t_m1 = 0, t_aa = 0, t_a0 = 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(ctrl + kBarFull + 8 * s, 1);
      mbar_init(ctrl + kBarEmpty + 8 * s, 1);
    }
    for (int c = 0; c < 8; ++c) {
      mbar_init(ctrl + kBarAFull + 8 * c, 1);
      mbar_init(ctrl + kBarAFree + 8 * c, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(ctrl + kBarOutFull + 8 * b, 1);
      mbar_init(ctrl + kBarOutFree + 8 * b, 16);  // 8 element-wise warps x 2 CTAs
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
  PairTile t;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (whole warp, elected lane)
    const uint32_t leader_full0 = mapa_u32(ctrl + kBarFull, 0), leader_a_full0 = mapa_u32(ctrl + kBarAFull, 0);
    uint32_t it = 0, segs = 0;  // ring stages issued / (chunk, pass) segments started, over all tiles
    bool ok = true;
    for (int n = 0; ok; ++n) {
      const int idx = tq_fetch(tq, n, true, abort_flag, p.status);
      if (idx < 0 || idx >= total_tiles) break;
      if (!pds2_decode(p, ppu, idx, t) || t.n_steps == 0) continue;
      const int rt_ld = min(2 * t.tp + rank, t.n_row_tiles - 1);  // clamped when the last pair has one tile
      const int apos = t.q_off + rt_ld * ppp;
      const int qb = g.cu_q ? 0 : t.b, kb = g.cu_k ? 0 : t.b;
      for (int c0 = 0; c0 < t.n_steps && ok; c0 += kChunkSteps) {
        const int c1 = min(c0 + kChunkSteps, t.n_steps);
        for (int mode = 0; mode < 2 && ok; ++mode, ++segs) {
          const CUtensorMap* tm_a = mode ? &tm_do : &tm_q;
          const CUtensorMap* tm_b = mode ? &tm_v : &tm_k;
          for (int j = c0; j < c1 && ok; ++j) {
            const int key0 = t.k_off + j * kStepKeys + rank * 128;
            for (int c = 0; c < 8 && ok; ++c) {
              if (j == c0) {
                // block c of this segment's A operand, as soon as the previous segment's last step has read
                // the old one
                if (segs > 0) {
                  ok = mbar_wait(ctrl + kBarAFree + 8 * c, (segs - 1) & 1, abort_flag, p.status, ST_TIMEOUT_LOAD);
                  ok = __all_sync(0xffffffffu, ok);
                  if (!ok) break;
                }
                if (elect_one()) {
                  if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarAFull + 8 * c, 2 * kABlockBytes);
                  tma_load_5d_pair(sA + c * kABlockBytes, tm_a, leader_a_full0 + 8 * c, c * 64, 0, apos, t.hu, qb);
                }
                __syncwarp();
              }
              const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
              ok = mbar_wait(ctrl + kBarEmpty + 8 * s, ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_LOAD);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) break;
              if (elect_one()) {
                if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarFull + 8 * s, 2 * kStageBytes);
                tma_load_4d_pair(sRing + s * kStageBytes, tm_b, leader_full0 + 8 * s, c * 64, key0, t.hkv, kb);
              }
              __syncwarp();
              ++it;
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA, whole warp)
    if (rank == 0) {
      constexpr uint32_t idesc = make_idesc(false, false, false, 256, kStepKeys);
      const uint32_t a_lo = desc_lo(sA, 16), ring_lo = desc_lo(sRing, 16);
      uint32_t it = 0, gs = 0, segs = 0;
      bool ok = true;
      const long long t_begin = prof ? clock64() : 0;
      for (int n = 0; ok; ++n) {
        const int idx = tq_fetch(tq, n, true, abort_flag, p.status);
        if (idx < 0 || idx >= total_tiles) break;
        if (!pds2_decode(p, ppu, idx, t) || t.n_steps == 0) continue;
        for (int c0 = 0; c0 < t.n_steps && ok; c0 += kChunkSteps) {
          const int c1 = min(c0 + kChunkSteps, t.n_steps);
          for (int mode = 0; mode < 2 && ok; ++mode, ++segs) {
            for (int j = c0; j < c1 && ok; ++j, ++gs) {
              const uint32_t b = gs & 1;
              if (gs >= 2) {  // buffer b must have been drained
                const long long t0 = prof ? clock64() : 0;
                ok = mbar_wait<true>(ctrl + kBarOutFree + 8 * b, ((gs >> 1) - 1) & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
                ok = __all_sync(0xffffffffu, ok);
                if (prof) t_b += clock64() - t0;
                if (!ok) break;
                tc_fence_after_sync();
              }
              const uint32_t d_tmem = tmem_base + b * 256;
              const bool last_step = j == c1 - 1;
#pragma unroll 1
              for (int c = 0; c < 8 && ok; ++c) {
                const long long t0 = prof ? clock64() : 0;
                if (j == c0) {  // this segment's block c of A has landed
                  ok = mbar_wait(ctrl + kBarAFull + 8 * c, segs & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
                  ok = __all_sync(0xffffffffu, ok);
                  if (!ok) break;
                  if (prof) t_aa += clock64() - t0;
                }
                const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                ok = mbar_wait(ctrl + kBarFull + 8 * s, ph, abort_flag, p.status, ST_TIMEOUT_MMA);
                ok = __all_sync(0xffffffffu, ok);
                if (prof) t_a += clock64() - t0;
                if (prof && j == c0) t_a0 += clock64() - t0;
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t a0 = a_lo + c * (kABlockBytes >> 4), b0 = ring_lo + s * (kStageBytes >> 4);
                if (elect_one()) {
#pragma unroll
                  for (int k = 0; k < 4; ++k)
                    umma_ss<2>(d_tmem, desc_join(a0 + ((k * 32) >> 4)), desc_join(b0 + ((k * 32) >> 4)), idesc, (c | k) != 0);
                  umma_commit_pair(ctrl + kBarEmpty + 8 * s, 3);
                  if (last_step) umma_commit_pair(ctrl + kBarAFree + 8 * c, 3);  // block c of A may be overwritten
                  if (c == 7) umma_commit_pair(ctrl + kBarOutFull + 8 * b, 3);
                }
                __syncwarp();
                ++it;
              }
            }
          }
        }
      }
      if (prof && lane == 0) {
        dbg[0] = static_cast<float>(t_a);
        dbg[1] = static_cast<float>(t_b);
        dbg[2] = static_cast<float>(clock64() - t_begin);
        dbg[3] = static_cast<float>(gs);
        dbg[16] = static_cast<float>(t_aa);  // of dbg[0]: waiting for the resident operand's blocks
        dbg[17] = static_cast<float>(t_a0);  // of dbg[0]: in the first step of a segment (A and B waits)
      }
    }
  } else if (warp == 3) {
    if (rank == 0 && lane == 0)
      tq_schedule(ctrl + kTileQ, p.tile_counters + kCounterPds, p.tile_counters + kCounterPdsDone, pair_id, n_pairs,
                  total_tiles, abort_flag, p.status);
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ element-wise warps
    // TMEM lane = row of the tile; warp & 3 selects the 32 lanes, (warp - 4) / 4 the 128-key half of the step.
    const int q = warp & 3, ch = (warp - 4) >> 2;
    const int L = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int64_t plane = p.ws_rows * p.ws_pitch;
    const uint32_t leader_free0 = mapa_u32(ctrl + kBarOutFree, 0);
    // P is read back by this kernel a few microseconds after it is written, dS not before the next kernel:
    // tell L2 which of the two to keep when it has to choose
    const uint64_t pol_keep = l2_policy_keep(), pol_stream = l2_policy_stream();
    bool ok = true;
    uint32_t gs = 0;
    const long long t_begin = prof ? clock64() : 0;
    for (int n = 0; ok; ++n) {
      const int idx = tq_fetch(tq, n, true, abort_flag, p.status);
      if (idx < 0 || idx >= total_tiles) break;
      if (!pds2_decode(p, ppu, idx, t) || t.n_steps == 0) continue;
      const int rt = 2 * t.tp + rank;
      const bool tile_valid = rt < t.n_row_tiles;  // the last pair of a sequence may hold one tile only
      const int pos = rt * ppp + L / g.pack_g;
      const int head = (g.pack_g > 1) ? t.hu * g.pack_g + L % g.pack_g : t.hu;
      const bool row_ok = tile_valid && pos < t.sq;
      int limit = t.sk - 1;
      if (g.causal) limit = min(limit, pos + t.sk - t.sq);
      if (!row_ok) limit = -1;
      // pass 0 stores P * 2^14, pass 1 stores dS * 2^e (bwd_common.cuh); both factors are folded into constants:
      //   P'  = exp2(S * scale_log2 - (lse_log2 - 14))
      //   t'  = (dP - dpsum) * scale * 2^(e - 14)  (fp16),   dS' = P' * t'  (one packed fp16 multiply)
      float lse2 = 0.f, t_mul = 0.f, t_add = 0.f;
      if (row_ok) {
        const int64_t ridx = g.cu_q ? static_cast<int64_t>(head) * p.total_q + t.q_off + pos
                                    : (static_cast<int64_t>(t.b) * g.heads_q + head) * t.sq + pos;
        const int e = ds_exponent(p.stats + static_cast<int64_t>(t.b * g.heads_kv + t.hkv) * kStatWords, p.scale);
        lse2 = p.lse_log2[ridx] - static_cast<float>(kPShift);
        t_mul = p.scale * pow2i(e - kPShift);
        t_add = -p.dpsum[ridx] * t_mul;
      }
      // this thread's row in the P plane; the dS plane is `plane` elements further
      uint16_t* ws_row = p.ws + (static_cast<int64_t>(t.hu - p.c_hu0) * 2) * plane +
                         (chunk_ws_row(p, t.tile_base, min(rt, t.n_row_tiles - 1)) + L) * p.ws_pitch;
      // after the 4 x 4 chunk transposes a thread handles chunk (lane & 3) of rows (lane & ~3) + r, r = 0..3
      const int64_t row_delta0 = static_cast<int64_t>((lane & ~3) - lane) * p.ws_pitch;

      // pass 1: the P values of a step come back with the access pattern of the stores (lane l reads 32-byte
      // chunk l & 3 of rows (l & ~3) + r: whole 128-byte lines per instruction, a quarter of the L1 wavefronts
      // of own-row loads) and are used in that layout. The values were stored by lanes of this same warp a chunk
      // of steps ago (__syncwarp orders the two) and normally still sit in L2. Each 64-key half is re-loaded for
      // the NEXT step as soon as this step is done with it, so the latency of the loads hides behind the rest of
      // the step.
      uint32_t pq[64];
      auto load_p_half = [&](int step, int h2) {
        const uint16_t* src = ws_row + row_delta0 + step * kStepKeys + ch * 128 + h2 * 64 + (lane & 3) * 16;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          if (tile_valid)
            ld_global_v8_hint(src + r * p.ws_pitch, &pq[h2 * 32 + 8 * r], pol_stream);  // read once: may go now
          else
#pragma unroll
            for (int i = 0; i < 8; ++i) pq[h2 * 32 + 8 * r + i] = 0u;
        }
      };
      for (int c0 = 0; c0 < t.n_steps && ok; c0 += kChunkSteps) {
        const int c1 = min(c0 + kChunkSteps, t.n_steps);
        for (int mode = 0; mode < 2 && ok; ++mode) {
          if (mode == 1) {
            __syncwarp();  // the P stores of this chunk (other lanes of this warp) before the loads below
            load_p_half(c0, 0);
            load_p_half(c0, 1);
          }
          for (int j = c0; j < c1 && ok; ++j, ++gs) {
            const uint32_t b = gs & 1;
            const int key_base = j * kStepKeys + ch * 128;
            const long long t0 = prof ? clock64() : 0;
            ok = mbar_wait(ctrl + kBarOutFull + 8 * b, (gs >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
            const long long t1 = prof ? clock64() : 0;
            if (prof) t_c += t1 - t0;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              uint32_t s[64];
              const uint32_t addr = lane_addr + b * 256 + ch * 128 + h2 * 64;
              tmem_ld32(addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
              tmem_ld32(addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
              tmem_ld_wait();
              if (h2 == 1) {  // the buffer has been read: hand it back to the tensor pipe
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(leader_free0 + 8 * b);
              }
              const int key0 = key_base + h2 * 64;
              const int cl = limit - key0;  // columns > cl are masked
              uint32_t x[32];
              const bool full = __all_sync(0xffffffffu, cl >= 63);  // warp-uniform fast path without masks
              if (mode == 0) {
                if (full) {
#pragma unroll
                  for (int i = 0; i < 64; i += 2)
                    x[i >> 1] = pack_half2(ex2(fmaf(__uint_as_float(s[i]), p.scale_log2, -lse2)),
                                           ex2(fmaf(__uint_as_float(s[i + 1]), p.scale_log2, -lse2)));
                } else {
#pragma unroll
                  for (int i = 0; i < 64; i += 2) {
                    const float a = ex2(fmaf(__uint_as_float(s[i]), p.scale_log2, -lse2));
                    const float bb = ex2(fmaf(__uint_as_float(s[i + 1]), p.scale_log2, -lse2));
                    x[i >> 1] = pack_half2(i > cl ? 0.f : a, i + 1 > cl ? 0.f : bb);
                  }
                }
                transpose_chunks32_4x4(x, lane);
              } else {
                // t' of this thread's own row, packed to fp16, goes through the SAME 4 x 4 chunk transpose as the
                // stores; P' was loaded in that layout already, so dS' is one packed multiply per register and
                // nothing has to be transposed back.
                if (full) {
#pragma unroll
                  for (int i = 0; i < 64; i += 2)
                    x[i >> 1] = pack_half2(fmaf(__uint_as_float(s[i]), t_mul, t_add),
                                           fmaf(__uint_as_float(s[i + 1]), t_mul, t_add));
                } else {
                  // masked entries: P' is 0 there already; t' = 0 guards against non-finite dP of rows / keys
                  // outside the sequence (0 * inf)
#pragma unroll
                  for (int i = 0; i < 64; i += 2) {
                    const float a = fmaf(__uint_as_float(s[i]), t_mul, t_add);
                    const float bb = fmaf(__uint_as_float(s[i + 1]), t_mul, t_add);
                    x[i >> 1] = pack_half2(i > cl ? 0.f : a, i + 1 > cl ? 0.f : bb);
                  }
                }
                transpose_chunks32_4x4(x, lane);
#pragma unroll
                for (int w = 0; w < 32; ++w) x[w] = mul_half2(x[w], pq[h2 * 32 + w]);
                if (j + 1 < c1) load_p_half(j + 1, h2);  // these registers are free again: next step's P
              }
              // 64 keys x 2 bytes = 4 chunks of 32 bytes per row; after the transpose every 256-bit store
              // instruction of the warp writes whole 128-byte lines
              if (tile_valid) {
                uint16_t* dst = ws_row + (mode ? plane : 0) + row_delta0 + key0 + (lane & 3) * 16;
#pragma unroll
                for (int r = 0; r < 4; ++r) st_global_v8_hint(dst + r * p.ws_pitch, &x[8 * r], mode ? pol_stream : pol_keep);
              }
            }
            if (prof) (mode ? t_m1 : t_m0) += clock64() - t1;
          }
        }
      }
    }
    if (prof && warp == 4 && lane == 0) {
      dbg[4] = static_cast<float>(t_c);
      dbg[5] = static_cast<float>(clock64() - t_begin);
      dbg[6] = static_cast<float>(t_m0);  // busy cycles of the P steps / of the dS steps
      dbg[7] = static_cast<float>(t_m1);
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

int launch_bwd_pds(const splitd_params* p, const BwdPlan& pl, int chunk, cudaStream_t stream) {
  BwdParams bp;
  if (int e = fill_bwd_params(p, bp, &pl)) return e;
  plan_chunk(pl, chunk, p, bp);
  const TileGeom& g = bp.g;
  CUtensorMap tm_q, tm_do, tm_k, tm_v;
  if (int e = make_q_tmap(&tm_q, p->q, p, g, p->q_strides, 2 * g.pos_per_cta, "q")) return e;
  if (int e = make_q_tmap(&tm_do, p->dout, p, g, p->do_strides, 2 * g.pos_per_cta, "dout")) return e;
  if (int e = make_kv_tmap(&tm_k, p->k, p, p->k_strides, 128, "k")) return e;
  if (int e = make_kv_tmap(&tm_v, p->v, p, p->v_strides, 128, "v")) return e;
  const bool varlen = p->cu_seqlens_q != nullptr;
  const int ppu = varlen ? (g.row_tiles + g.batch + 1) / 2 : (g.row_tiles + 1) / 2;
  const long long nhu = bp.c_hu1 - bp.c_hu0;
  const long long pairs = varlen ? static_cast<long long>(ppu) * nhu : static_cast<long long>(bp.c_ntp) * bp.c_nb * nhu;
  if (pairs <= 0 || pairs > (1ll << 30)) return fail(SPLITD_ERR_INVALID_ARGUMENT, "P/dS grid out of range");
  static std::atomic<int> cache[64];
  const int resident = resident_cluster_pairs(splitd_bwd_pds2_kernel, pds2::kThreads, pds2::kSmemBytes, cache);
  if (resident <= 0) return fail(SPLITD_ERR_CUDA, "cudaFuncSetAttribute(P/dS kernel) failed");
  const long long grid_pairs = pairs < resident ? pairs : resident;
  splitd_bwd_pds2_kernel<<<dim3(static_cast<unsigned>(2 * grid_pairs)), dim3(pds2::kThreads), pds2::kSmemBytes,
                           stream>>>(tm_q, tm_do, tm_k, tm_v, bp, static_cast<int>(pairs), ppu);
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "P/dS launch failed: %s", cudaGetErrorString(ce));
  return 0;
}

}  // namespace sd
