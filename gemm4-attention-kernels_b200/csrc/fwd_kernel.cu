// Forward kernel: O = softmax(Q K^T * scale [+causal]) V and LSE for head_dim 512 on sm_100a.
//
// A 128 x 512 fp32 output tile fills all 512 TMEM columns of one SM, so a tile of 128 packed query
// rows is split over a CTA PAIR and every GEMM is a cta_group::2 UMMA with M = 128 (64 rows per
// CTA). In that shape each CTA's 64 x N accumulator uses all 128 TMEM lanes with N/2 columns
// (lanes 0-63 hold columns [0,N/2), lanes 64-127 hold [N/2,N)), so per CTA
//     O (64 x 512)           -> 2 accumulators x 128 columns   = columns [0,256)
//     S (64 x 256 keys) x 2  -> 2 buffers x 128 columns        = columns [256,512)
// and the B operand of every MMA (K rows for QK^T, V columns for PV) is split between the two
// CTAs, which halves the K/V bytes each SM pulls from L2.
// (Measured: this 64-rows-per-CTA form runs a 64 x 256 x 16 MMA in 64 cycles, i.e. at full rate, provided
// the issuing warp keeps up: see the MMA issuer below.)
//
// Per KV step of 256 keys:  S = Q K^T (32 MMAs, K-major operands)  ->  softmax warps: row max
// (exchanged between the four threads that share a row), P = exp2(...) as fp16 into shared memory
// -> O += P V (32 MMAs, V as MN-major B operand). P is fp16 for bf16 inputs too: with bf16's 8 significant
// bits the rounding of P alone puts a non-causal output at up to twice the error of a result that is rounded
// once; fp16 has 11. The two operands of an MMA must share a format, so for bf16 inputs V is read from an fp16
// copy that a small kernel makes in the caller's workspace right before (K/V are the small tensors of GQA).  S is double buffered so the tensor pipe runs
// S(j+1) while the softmax warps work on S(j).  O is only rescaled when a row max grows by more
// than 2^8 (the exact value is restored by the final 1/rowsum scaling).
//
// PERSISTENT pairs: the grid is one pair per SM pair; each pair walks over tiles (snake order over the
// tile list, whose blocks alternate between heaviest-first and lightest-first under a causal mask: that keeps
// pairs balanced and keeps concurrently running pairs on the same K/V). Shared memory is six 32 KB slots + a 32 KB P buffer: a tile's Q occupies two slots, the K/V
// ring four. Q is loaded like any other ring entry, so the NEXT tile's Q arrives in the first two ring
// slots that the current tile's last PV frees, and at the tile switch the old Q slots join the ring: no
// idle time for launch, TMEM allocation, barrier set-up or the Q load between tiles, and the epilogue of
// one tile overlaps the first two QK^T products of the next.
//
// Warp roles (384 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only) + TMEM
// allocation, warps 4-11 softmax / epilogue: two warps per TMEM lane quarter, each thread owning 64
// of the 128 S columns of its lane. Follows the math of the reference forward
// (src/flash_fwd_sm90_d512.py:921-1222, src/softmax.py:48-135) with a different decomposition.
#include <cstring>

#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"
#include "rowcopy.cuh"

namespace sd {

namespace fwd {
constexpr int kStepKeys = 256;                 // keys per KV step (UMMA N)
constexpr int kStages = 4;                     // logical ring stages
constexpr int kSlots = 6;                      // physical 32 KB slots: 4 ring + 2 Q
constexpr int kStageBytes = 32768;
constexpr int kOffSlots = 0;
constexpr int kOffP = kSlots * kStageBytes;    // 32 KB P buffer
constexpr int kOffCtrl = kOffP + 32768;
// control block layout (bytes from kOffCtrl)
constexpr int kBarFull = 0;                        // [kStages]
constexpr int kBarEmpty = kBarFull + 8 * kStages;  // [kStages]
constexpr int kBarSFull = kBarEmpty + 8 * kStages; // [2]
constexpr int kBarPFull = kBarSFull + 16;
constexpr int kBarPvDone = kBarPFull + 8;
constexpr int kBarOFree = kBarPvDone + 8;
constexpr int kBarXchg = kBarOFree + 8;            // [2] one per partner-warp set
constexpr int kTmemPtr = kBarXchg + 16;
constexpr int kAbort = kTmemPtr + 4;
constexpr int kXchg = 192;                         // float [2][256]
constexpr int kCtrlBytes = kXchg + 2 * 256 * 4;
constexpr int kSmemBytes = kOffCtrl + kCtrlBytes;  // the dynamic segment is 1024-byte aligned (checked)
static_assert(kAbort + 4 <= kXchg, "control block overlap");
static_assert(kSmemBytes <= 232448, "shared memory budget");
constexpr int kTmemColsO = 0;
constexpr int kTmemColsS = 256;
constexpr float kRescaleThreshold = 8.0f;          // log2 units
// A row whose largest probability exceeds this keeps the low word of its output for the backward (rows whose
// probability mass sits on few keys have |out| ~ |v|, where the 16-bit rounding of out matters; below the
// threshold the mass is spread over at least 16 keys)
constexpr float kResidPmax = 1.f / 16.f;
}  // namespace fwd

// Slot tables kept in registers: nibble s of `tab` is the physical slot of logical ring stage s.
__device__ __forceinline__ uint32_t slot_get(uint32_t tab, uint32_t s) { return (tab >> (4 * s)) & 15u; }
__device__ __forceinline__ uint32_t slot_set(uint32_t tab, uint32_t s, uint32_t v) {
  return (tab & ~(15u << (4 * s))) | (v << (4 * s));
}

// Tile slot visited by pair `pair` in round r (snake order). Returns false when the slot index is past
// the end; `valid` says whether the slot holds a tile (the packed layout over-counts slots).
__device__ __forceinline__ bool fwd_next_tile(const FwdParams& p, int r, int pair, int n_pairs, TileCoord& tc,
                                              int& step0, int& n_steps, bool& valid, int* last_chunks = nullptr) {
  if (static_cast<long long>(r) * n_pairs >= p.total_pairs) return false;
  const int idx = r * n_pairs + ((r & 1) ? n_pairs - 1 - pair : pair);
  valid = idx < p.total_pairs && decode_tile(p.g, idx, tc);
  step0 = 0;
  n_steps = 0;
  if (valid && p.g.causal) {
    // decode_tile lists the row tiles of every (batch, head unit) block heaviest first. Walk every other block
    // lightest first instead (the last block of the list always heaviest first): the weights along the list
    // then have no jumps at the block borders, which is what the static round-robin assignment of the list to
    // the pairs needs to come out balanced. With a jump, the pairs that draw the light end of one block in
    // the round that crosses the border stay a heavy tile behind the others for good: 3-5 % at S >= 4096.
    const int blk = p.g.cu_q ? tc.hu * p.g.batch + tc.b : tc.b * p.g.head_units + tc.hu;
    if ((p.g.batch * p.g.head_units - 1 - blk) & 1) {
      const int pos_per_pair = 2 * p.g.pos_per_cta;
      const int nt = (tc.sq + pos_per_pair - 1) / pos_per_pair;
      const int rt = nt - 1 - tc.rt;
      tc.tile_global += rt - tc.rt;
      tc.rt = rt;
      tc.p0 = rt * pos_per_pair;
    }
  }
  if (valid) {
    // keys visible to row i: [i + sk - sq - win_left, i + sk - sq + win_right] (each side optional)
    int kv_hi = tc.sk, kv_lo = 0;
    if (p.win_right >= 0) {
      const int last_pos = min(tc.p0 + 2 * p.g.pos_per_cta, tc.sq) - 1;
      kv_hi = min(kv_hi, last_pos + 1 + tc.sk - tc.sq + p.win_right);
    }
    if (p.win_left >= 0) kv_lo = max(0, tc.p0 + tc.sk - tc.sq - p.win_left);
    if (kv_hi > kv_lo) {
      step0 = kv_lo / fwd::kStepKeys;
      n_steps = (kv_hi + fwd::kStepKeys - 1) / fwd::kStepKeys - step0;
      // P is zero for every row of the tile beyond kv_hi: the last step's PV only needs this many 64-key chunks
      if (last_chunks) *last_chunks = (kv_hi - (step0 + n_steps - 1) * fwd::kStepKeys + 63) / 64;
    }
  }
  return true;
}

// A tile with at least one KV step, as the producer and the MMA issuer see it.
struct FwdWork {
  TileCoord tc;
  int r, step0, n_steps, last_chunks;
};

// First round >= r_from in which this pair has a tile with work; false when the pair's list is exhausted.
__device__ __forceinline__ bool fwd_find_work(const FwdParams& p, int r_from, int pair, int n_pairs, FwdWork& w) {
  bool valid;
  w.last_chunks = 4;
  for (int r = r_from; fwd_next_tile(p, r, pair, n_pairs, w.tc, w.step0, w.n_steps, valid, &w.last_chunks); ++r) {
    if (valid && w.n_steps > 0) {
      w.r = r;
      return true;
    }
  }
  return false;
}

template <bool kFp16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(384, 1)
splitd_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                  const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using namespace fwd;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t smem_base = smem_u32(smem_raw);
  uint8_t* smem = smem_raw;
  if (smem_base & 1023u) {  // swizzled tiles need 1024-byte aligned bases
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, ST_BAD_SMEM_ALIGN);
    return;
  }
  const uint32_t sSlots = smem_base + kOffSlots, sP = smem_base + kOffP;
  const uint32_t ctrl = smem_base + kOffCtrl;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffCtrl + kAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kOffCtrl + kTmemPtr);
  float* xchg = reinterpret_cast<float*>(smem + kOffCtrl + kXchg);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const TileGeom& g = p.g;

  // per-role cycle counters of pair 0, written to debug[32..51]; compiled in with -DSPLITD_PROFILE only
  const bool prof = kProfile && p.debug != nullptr && pair_id == 0 && rank == 0;
  long long t_a = 0, t_b = 0, t_c = 0, t_all = 0;

  // ---------------------------------------------------------------- setup (once per pair)
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(ctrl + kBarFull + 8 * s, 1);
      mbar_init(ctrl + kBarEmpty + 8 * s, 1);
    }
    mbar_init(ctrl + kBarSFull, 1);
    mbar_init(ctrl + kBarSFull + 8, 1);
    mbar_init(ctrl + kBarPFull, 16);  // 8 softmax warps x 2 CTAs
    mbar_init(ctrl + kBarPvDone, 1);
    mbar_init(ctrl + kBarOFree, 16);
    mbar_init(ctrl + kBarXchg, 128);
    mbar_init(ctrl + kBarXchg + 8, 128);
    fence_mbar_init();
    prefetch_tmap(&tm_q);
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
  const uint32_t leader_p_full = mapa_u32(ctrl + kBarPFull, 0);
  const uint32_t leader_o_free = mapa_u32(ctrl + kBarOFree, 0);

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // Like the MMA issuer below, the whole warp runs the loop and one elected lane issues the copies: the
    // warp-uniform form spends about half the cycles per stage of a single lane under a divergent branch,
    // and every cycle this warp is busy is a cycle a freed ring slot waits for its next load.
    {
      uint32_t it = 0;      // ring acquisitions so far (Q takes two per tile)
      bool ok = true;
      uint32_t rs = 0x3210u;  // logical ring stage -> physical slot (one nibble each)
      uint32_t qs = 0x54u;    // slots that held the previous tile's Q (free at the start)
      const uint32_t leader_full0 = mapa_u32(ctrl + kBarFull, 0);
      // wait for the stage's slot with all lanes (warp-uniform outcome); the elected lane arms the barrier
      auto acquire = [&](uint32_t& st, uint32_t& bar, uint32_t& stage) {
        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
        const long long t0 = prof ? clock64() : 0;
        if (ok) {
          ok = mbar_wait(ctrl + kBarEmpty + 8 * s, ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_LOAD);
          ok = __all_sync(0xffffffffu, ok);
        }
        if (prof) t_a += clock64() - t0;
        st = sSlots + slot_get(rs, s) * kStageBytes;
        bar = leader_full0 + 8 * s;
        stage = s;
        ++it;
      };
      const long long tp0 = prof ? clock64() : 0;
      // Q: two ring acquisitions (4 D blocks of 8 KB each) that stay resident for the whole tile
      auto load_q = [&](const FwdWork& w) {
        const int qpos = w.tc.q_off + w.tc.p0 + static_cast<int>(rank) * g.pos_per_cta;
        const int qb = g.cu_q ? 0 : w.tc.b;
        uint32_t newq = 0;
        for (int u = 0; u < 2 && ok; ++u) {
          uint32_t st, bar, stage;
          acquire(st, bar, stage);
          if (!ok) break;
          if (elect_one()) {
            if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarFull + 8 * stage, 2 * kStageBytes);
#pragma unroll
            for (int d = 0; d < 4; ++d)
              tma_load_5d_pair(st + d * 8192, &tm_q, bar, (u * 4 + d) * 64, 0, qpos, w.tc.hu, qb);
          }
          __syncwarp();
          newq = slot_set(newq, u, slot_get(rs, stage));
          rs = slot_set(rs, stage, slot_get(qs, u));  // the previous tile's Q slot joins the ring here
        }
        qs = newq;
      };
      // this CTA's 128 key rows of a step (first key `key`), 128 of the 512 D columns per stage
      auto load_k = [&](int b, int hkv, int key) {
        const int kb = g.cu_k ? 0 : b;
        const int key0 = key + static_cast<int>(rank) * 128;
        for (int c = 0; c < 4 && ok; ++c) {
          uint32_t st, bar, stage;
          acquire(st, bar, stage);
          if (!ok) break;
          if (elect_one()) {
            if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarFull + 8 * stage, 2 * kStageBytes);
            tma_load_4d_pair(st, &tm_k, bar, (2 * c) * 64, key0, hkv, kb);
            tma_load_4d_pair(st + 16384, &tm_k, bar, (2 * c + 1) * 64, key0, hkv, kb);
          }
          __syncwarp();
        }
      };
      auto load_v = [&](const FwdWork& w, int j) {  // 64 keys per stage, this CTA's 2 x 128 V columns (both accumulators)
        const int kb = g.cu_k ? 0 : w.tc.b;
        const int n_kq = j == w.n_steps - 1 ? w.last_chunks : 4;
        for (int kq = 0; kq < n_kq && ok; ++kq) {
          uint32_t st, bar, stage;
          acquire(st, bar, stage);
          if (!ok) break;
          const int key0 = w.tc.k_off + (w.step0 + j) * kStepKeys + kq * 64;
          if (elect_one()) {
            if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarFull + 8 * stage, 2 * kStageBytes);
#pragma unroll
            for (int m = 0; m < 2; ++m) {
              const int dv0 = m * 256 + static_cast<int>(rank) * 128;
              tma_load_4d_pair(st + m * 16384, &tm_v, bar, dv0, key0, w.tc.hkv, kb);
              tma_load_4d_pair(st + m * 16384 + 8192, &tm_v, bar, dv0 + 64, key0, w.tc.hkv, kb);
            }
          }
          __syncwarp();
        }
      };
      // Ring order = the MMA issuer's order: the operands of the NEXT QK^T product (of this tile, or Q and the
      // first K step of the next tile) go in front of the V rows of the current step.
      FwdWork cur, nxt;
      bool have = fwd_find_work(p, 0, pair_id, n_pairs, cur);
      if (have) {
        load_q(cur);
        load_k(cur.tc.b, cur.tc.hkv, cur.tc.k_off + cur.step0 * kStepKeys);
      }
      while (have && ok) {
        const bool has_next = fwd_find_work(p, cur.r + 1, pair_id, n_pairs, nxt);
        for (int j = 0; j < cur.n_steps && ok; ++j) {
          if (j + 1 < cur.n_steps) {
            load_k(cur.tc.b, cur.tc.hkv, cur.tc.k_off + (cur.step0 + j + 1) * kStepKeys);
          } else if (has_next) {
            load_q(nxt);
            load_k(nxt.tc.b, nxt.tc.hkv, nxt.tc.k_off + nxt.step0 * kStepKeys);
          }
          load_v(cur, j);
        }
        cur = nxt;
        have = has_next;
      }
      if (prof && lane == 0) {
        p.debug[32] = static_cast<float>(t_a);
        p.debug[33] = static_cast<float>(clock64() - tp0);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA)
    // The WHOLE warp runs this loop and one elected lane issues: with warp-uniform control flow the barrier
    // waits, descriptor arithmetic and commits cost ~42 cycles per MMA, which keeps the 64-cycle MMAs of this
    // shape back to back; the same loop run by a single lane under a divergent branch costs ~85 cycles per
    // MMA (both measured). Descriptor low words are advanced by adding, the high word is a constant, and one
    // barrier wait / commit covers 8 MMAs (a 32 KB stage).
    if (rank == 0) {
      constexpr uint32_t idesc_s = make_idesc(kFp16, false, false, 128, kStepKeys);
      constexpr uint32_t idesc_pv = make_idesc(true, false, true, 128, 256);  // P and V (copy) are fp16 always
      const uint32_t p_lo = desc_lo(sP, 16);
      uint32_t it = 0;     // ring acquisitions consumed
      uint32_t gs = 0;     // KV steps issued so far (S buffer / barrier phase index)
      uint32_t tiles = 0;  // tiles with work done so far
      uint32_t rs = 0x3210u, qs = 0x54u;  // same slot tables as the producer's
      bool ok = true;
      t_all = kProfile && p.debug != nullptr ? clock64() : 0;
      // wait on a barrier with all lanes, keep the outcome warp-uniform
      auto wait_all = [&](uint32_t bar, uint32_t parity, bool cluster_scope) {
        bool w = cluster_scope ? mbar_wait<true>(bar, parity, abort_flag, p.status, ST_TIMEOUT_MMA)
                               : mbar_wait(bar, parity, abort_flag, p.status, ST_TIMEOUT_MMA);
        return __all_sync(0xffffffffu, w);
      };
      uint32_t q_lo[2] = {0, 0};
      // Q of a tile: wait for its two ring entries, hand the previous tile's Q slots to the ring
      auto take_q = [&]() {
        uint32_t newq = 0;
        for (int u = 0; u < 2 && ok; ++u) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          ok = wait_all(ctrl + kBarFull + 8 * s, ph, false);
          if (!ok) return;
          newq = slot_set(newq, u, slot_get(rs, s));
          rs = slot_set(rs, s, slot_get(qs, u));
          if (elect_one()) umma_commit_pair(ctrl + kBarEmpty + 8 * s, 3);  // old Q slot is free once all earlier MMAs are done
          __syncwarp();
          ++it;
        }
        qs = newq;
        q_lo[0] = desc_lo(sSlots + slot_get(qs, 0) * kStageBytes, 16);
        q_lo[1] = desc_lo(sSlots + slot_get(qs, 1) * kStageBytes, 16);
      };
      auto issue_s = [&](uint32_t step) {
        const uint32_t d_tmem = tmem_base + kTmemColsS + (step & 1) * 128;
#pragma unroll 1
        for (int c = 0; c < 4 && ok; ++c) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          const long long t0 = prof ? clock64() : 0;
          ok = wait_all(ctrl + kBarFull + 8 * s, ph, false);
          if (prof) t_a += clock64() - t0;
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a0 = (c < 2 ? q_lo[0] : q_lo[1]) + (((c & 1) * 16384) >> 4);
          const uint32_t b0 = desc_lo(sSlots + slot_get(rs, s) * kStageBytes, 16);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint32_t offa = ((k >> 2) * 8192 + (k & 3) * 32) >> 4;   // A: 8 KB per 64-wide D block
              const uint32_t offb = ((k >> 2) * 16384 + (k & 3) * 32) >> 4;  // B: 16 KB per 64-wide D block
              umma_ss<2>(d_tmem, desc_join(a0 + offa), desc_join(b0 + offb), idesc_s, (c | k) != 0);
            }
            umma_commit_pair(ctrl + kBarEmpty + 8 * s, 3);
            if (c == 3) umma_commit_pair(ctrl + kBarSFull + 8 * (step & 1), 3);
          }
          __syncwarp();
          ++it;
        }
      };
      auto issue_pv = [&](int j, int n_kq) {
#pragma unroll 1
        for (int kq = 0; kq < n_kq && ok; ++kq) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          const long long t0 = prof ? clock64() : 0;
          ok = wait_all(ctrl + kBarFull + 8 * s, ph, false);
          if (prof) t_b += clock64() - t0;
          if (!ok) break;
          tc_fence_after_sync();
          const uint32_t a0 = p_lo + kq * (8192 >> 4);
          const uint32_t b0 = desc_lo(sSlots + slot_get(rs, s) * kStageBytes, 8192);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
#pragma unroll
              for (int m = 0; m < 2; ++m)
                umma_ss<2>(tmem_base + kTmemColsO + m * 128, desc_join(a0 + ((k * 32) >> 4)),
                           desc_join(b0 + ((m * 16384 + k * 2048) >> 4)), idesc_pv, (j | kq | k) != 0);
            }
            umma_commit_pair(ctrl + kBarEmpty + 8 * s, 3);
            if (kq == n_kq - 1) umma_commit_pair(ctrl + kBarPvDone, 3);
          }
          __syncwarp();
          ++it;
        }
      };
      // Every iteration issues the NEXT QK^T product first (the next step of this tile, or the first step of
      // the pair's next tile) and then the PV product of the current step, so the softmax warps always find
      // the next scores ready and the tensor pipe has work while they are busy, across tile switches too.
      FwdWork cur, nxt;
      bool have = fwd_find_work(p, 0, pair_id, n_pairs, cur);
      if (have) {
        take_q();
        if (ok) issue_s(gs);
      }
      while (have && ok) {
        const bool has_next = fwd_find_work(p, cur.r + 1, pair_id, n_pairs, nxt);
        for (int j = 0; j < cur.n_steps && ok; ++j) {
          if (j + 1 < cur.n_steps) {
            issue_s(gs + 1);
          } else if (has_next) {
            take_q();
            if (ok) issue_s(gs + 1);
          }
          if (!ok) break;
          const long long t0 = prof ? clock64() : 0;
          ok = wait_all(ctrl + kBarPFull, gs & 1, true);
          if (ok && j == 0 && tiles > 0)  // the previous tile's epilogue must have drained O
            ok = wait_all(ctrl + kBarOFree, (tiles - 1) & 1, true);
          if (prof) t_c += clock64() - t0;
          if (!ok) break;
          tc_fence_after_sync();
          issue_pv(j, j == cur.n_steps - 1 ? cur.last_chunks : 4);
          ++gs;
        }
        ++tiles;
        cur = nxt;
        have = has_next;
      }
      // longest-running pair of the launch in units of 1024 cycles, as an integer in debug[35]
      if (kProfile && p.debug != nullptr && lane == 0)
        atomicMax(reinterpret_cast<int*>(p.debug + 35), static_cast<int>((clock64() - t_all) >> 10));
      if (prof && lane == 0) {
        p.debug[34] = static_cast<float>(gs);
        p.debug[36] = static_cast<float>(t_a);
        p.debug[37] = static_cast<float>(t_b);
        p.debug[38] = static_cast<float>(t_c);
        p.debug[39] = static_cast<float>(clock64() - t_all);
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax + epilogue
    const int q = warp & 3, wg = (warp - 4) >> 2;
    const int L = q * 32 + lane;            // TMEM lane of this thread
    const int row = L & 63, half = L >> 6;  // row within the CTA, which half of the N columns
    const int xi = wg * 128 + L;            // slot in the exchange arrays
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t xbar = ctrl + kBarXchg + 8 * (q & 1);
    const int grp_row0 = row & ~3;          // first row of this lane's group of 4 (epilogue stores)
    const int pack_shift = 31 - __clz(g.pack_g);  // heads fold into rows only when the group is a power of two
    uint32_t xphase = 0;
    uint32_t gs = 0;                        // KV steps seen so far (same counter as the MMA issuer's)
    bool ok = true;
    uint32_t r[64];
    TileCoord tc;
    int step0, n_steps;
    bool valid;
    t_all = prof ? clock64() : 0;
    long long tph0 = 0, tph1 = 0, tph2 = 0, tph3 = 0, tph4 = 0, tph5 = 0, tph6 = 0;

    // Epilogue of a tile: O / rowsum -> global memory, LSE. `has_acc` is false for a tile without visible keys
    // (zeros, LSE = -inf, no TMEM access). The caller has waited for the tile's last PV.
    auto epilogue = [&](int e_b, int e_hu, int e_p0, int e_sq, int e_qoff, float m_ref, float m_top, float l_sum,
                        bool has_acc) {
      const int pos = e_p0 + static_cast<int>(rank) * g.pos_per_cta + (row >> pack_shift);
      const int head = e_hu * g.pack_g + (row & (g.pack_g - 1));
      float l_tot = 0.f;
      if (has_acc) {
        // row sums of the four threads of a row
        float* xs = xchg + xphase * 256;
        xs[xi] = l_sum;
        mbar_arrive(xbar);
        ok = mbar_wait(xbar, xphase, abort_flag, p.status, ST_TIMEOUT_PEER);
        ok = __all_sync(0xffffffffu, ok);
        xphase ^= 1u;
        if (!ok) return;
        // one order of summation for the row's four threads: they must agree on the decision below
        l_tot = (xs[row] + xs[row + 64]) + (xs[row + 128] + xs[row + 192]);
      }
      const bool any = l_tot > 0.f;
      const float inv = any ? 1.f / l_tot : 0.f;
      // Low word of the output: written for a group of 4 rows (the 4 lanes that store together; the same rows in the
      // four warps that share them) when one of them is concentrated on few keys; a byte per row tells the backward
      // whether it is there.
      bool w_resid = false, g_resid = false;  // any group of the warp / this lane's group
      if (p.resid_rows != nullptr) {
        const bool peaked = any && (p.resid_all != 0 || ex2((m_top - m_ref) * p.scale_log2) * inv > kResidPmax);
        const uint32_t votes = __ballot_sync(0xffffffffu, peaked);
        w_resid = votes != 0u;
        g_resid = ((votes >> (lane & ~3)) & 0xfu) != 0u;
        if (pos < e_sq && half == 0 && wg == 0) {
          const int64_t idx = g.cu_q ? static_cast<int64_t>(head) * p.total_q + e_qoff + pos
                                     : (static_cast<int64_t>(e_b) * g.heads_q + head) * e_sq + pos;
          p.resid_flags[idx] = g_resid ? 1 : 0;
        }
      }
      if (pos < e_sq && half == 0 && wg == 0 && p.lse != nullptr) {
        const float ms = (m_ref == -INFINITY ? 0.f : m_ref) * p.scale_log2;
        const float lse = any ? (ms + lg2(l_tot)) * kLn2 : -INFINITY;
        const int64_t idx = g.cu_q ? static_cast<int64_t>(head) * p.total_q + e_qoff + pos
                                   : (static_cast<int64_t>(e_b) * g.heads_q + head) * e_sq + pos;
        p.lse[idx] = lse;
      }
      // Stores: each thread owns one row, so a plain store per thread would touch 32 different lines per warp
      // instruction. 4 x 4 transposes of 32-byte chunks inside groups of 4 lanes make every store instruction
      // write 8 full 128-byte lines instead. The four row addresses are computed once per tile.
      uint16_t* obase = reinterpret_cast<uint16_t*>(p.o) + (g.cu_q ? 0 : e_b * p.o_stride_b) + wg * 256 + half * 128 +
                        (lane & 3) * 16;
      uint16_t* rowp[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int re = grp_row0 + e;
        const int pos_e = e_p0 + static_cast<int>(rank) * g.pos_per_cta + (re >> pack_shift);
        const int head_e = e_hu * g.pack_g + (re & (g.pack_g - 1));
        rowp[e] = pos_e < e_sq ? obase + static_cast<int64_t>(e_qoff + pos_e) * p.o_stride_s +
                                     static_cast<int64_t>(head_e) * p.o_stride_h
                               : nullptr;
      }
      if (has_acc && !w_resid) {
        // The common case: read and pack both halves of the row first, so that O is handed back to the tensor pipe
        // (the next tile's first PV) before the transposes and the stores, not in the middle of them.
        uint32_t xa[32], xb[32];
        {
          uint32_t t[64];
          tmem_ld32(lane_addr + kTmemColsO + wg * 128, *reinterpret_cast<uint32_t(*)[32]>(&t[0]));
          tmem_ld32(lane_addr + kTmemColsO + wg * 128 + 32, *reinterpret_cast<uint32_t(*)[32]>(&t[32]));
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 64; i += 2)
            xa[i >> 1] = pack2<kFp16>(__uint_as_float(t[i]) * inv, __uint_as_float(t[i + 1]) * inv);
          tmem_ld32(lane_addr + kTmemColsO + wg * 128 + 64, *reinterpret_cast<uint32_t(*)[32]>(&t[0]));
          tmem_ld32(lane_addr + kTmemColsO + wg * 128 + 96, *reinterpret_cast<uint32_t(*)[32]>(&t[32]));
          tmem_ld_wait();
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive_remote(leader_o_free);
#pragma unroll
          for (int i = 0; i < 64; i += 2)
            xb[i >> 1] = pack2<kFp16>(__uint_as_float(t[i]) * inv, __uint_as_float(t[i + 1]) * inv);
        }
        transpose_chunks32_4x4(xa, lane);
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (rowp[e] != nullptr) st_global_32b(rowp[e], &xa[8 * e]);
        transpose_chunks32_4x4(xb, lane);
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (rowp[e] != nullptr) st_global_32b(rowp[e] + 64, &xb[8 * e]);
        return;
      }
#pragma unroll 1
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t t[64];
        if (has_acc) {
          tmem_ld32(lane_addr + kTmemColsO + wg * 128 + c2 * 64, *reinterpret_cast<uint32_t(*)[32]>(&t[0]));
          tmem_ld32(lane_addr + kTmemColsO + wg * 128 + c2 * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&t[32]));
          tmem_ld_wait();
          if (c2 == 1) {  // O has been read: the next tile's first PV may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(leader_o_free);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) t[i] = 0u;
        }
        // a row without a visible key has P = 0 throughout, so its accumulator is 0 and inv = 0 keeps it so
        uint32_t x[32];
#pragma unroll
        for (int i = 0; i < 64; i += 2)
          x[i >> 1] = pack2<kFp16>(__uint_as_float(t[i]) * inv, __uint_as_float(t[i + 1]) * inv);
        if (w_resid) {
          // low word: what the rounding of the output dropped, rounded to 16 bits itself (t is overwritten in place)
#pragma unroll
          for (int i = 0; i < 64; i += 2) {
            float h0, h1;
            unpack2<kFp16>(x[i >> 1], h0, h1);
            t[i >> 1] = pack2<kFp16>(fmaf(__uint_as_float(t[i]), inv, -h0), fmaf(__uint_as_float(t[i + 1]), inv, -h1));
          }
        }
        transpose_chunks32_4x4(x, lane);
        // now x[8e..8e+7] = 32-byte chunk (lane & 3) of row grp_row0 + e
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (rowp[e] != nullptr) st_global_32b(rowp[e] + c2 * 64, &x[8 * e]);
        if (w_resid) {
          uint32_t(&y)[32] = *reinterpret_cast<uint32_t(*)[32]>(&t[0]);
          transpose_chunks32_4x4(y, lane);
          // rows of the low word are contiguous, (batch, position, head, 512) / (token, head, 512)
          const int64_t tok0 = (g.cu_q ? 0 : static_cast<int64_t>(e_b) * e_sq) + e_qoff;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int re = grp_row0 + e;
            const int pos_e = e_p0 + static_cast<int>(rank) * g.pos_per_cta + (re >> pack_shift);
            const int head_e = e_hu * g.pack_g + (re & (g.pack_g - 1));
            if (g_resid && pos_e < e_sq)
              st_global_32b(p.resid_rows + ((tok0 + pos_e) * g.heads_q + head_e) * kHeadDim + wg * 256 + half * 128 +
                                (lane & 3) * 16 + c2 * 64,
                            &y[8 * e]);
          }
        }
      }
    };

    int prev_b = 0, prev_hu = 0, prev_p0 = 0, prev_sq = 0, prev_qoff = 0;  // what the owed epilogue needs of its tile
    float prev_m = 0.f, prev_mt = 0.f, prev_l = 0.f;
    bool have_prev = false;  // a tile whose steps are done but whose epilogue has not run yet
    long long t_epi = 0;

    for (int rr = 0; ok; ++rr) {
      const bool more = fwd_next_tile(p, rr, pair_id, n_pairs, tc, step0, n_steps, valid);
      if (more && !valid) continue;
      if (!more || n_steps == 0) {
        // End of the list, or a tile without a visible key: first the epilogue that is still owed, then
        // (for such a tile) zeros and LSE = -inf.
        if (have_prev) {
          ok = mbar_wait(ctrl + kBarPvDone, (gs - 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
          have_prev = false;
          epilogue(prev_b, prev_hu, prev_p0, prev_sq, prev_qoff, prev_m, prev_mt, prev_l, true);
        }
        if (more && ok) epilogue(tc.b, tc.hu, tc.p0, tc.sq, tc.q_off, -INFINITY, -INFINITY, 0.f, false);
        if (!more) break;
        continue;
      }
      const int pos = tc.p0 + static_cast<int>(rank) * g.pos_per_cta + (row >> pack_shift);
      int limit = tc.sk - 1;  // last visible key of this row
      if (p.win_right >= 0) limit = min(limit, pos + tc.sk - tc.sq + p.win_right);
      const int lo_limit = p.win_left >= 0 ? pos + tc.sk - tc.sq - p.win_left : 0;  // first visible key
      float m_ref = -INFINITY, m_top = -INFINITY, l_sum = 0.f;  // m_top: the row's largest score so far

      for (int j = 0; j < n_steps && ok; ++j, ++gs) {
        long long t0 = prof ? clock64() : 0;
        ok = mbar_wait(ctrl + kBarSFull + 8 * (gs & 1), (gs >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
        if (prof) t_a += clock64() - t0;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t s_addr = lane_addr + kTmemColsS + (gs & 1) * 128 + wg * 64;
        const int key0 = (step0 + j) * kStepKeys + half * 128 + wg * 64;  // key of this thread's column 0
        const int cl = limit - key0;                                       // columns > cl are masked
        const int cl_lo = lo_limit - key0;                                 // columns < cl_lo are masked

        long long q0 = prof ? clock64() : 0;
        tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_ld_wait();
        if (prof) { r[0] = __float_as_uint(__uint_as_float(r[0]) + 0.f); const long long q1 = clock64(); tph0 += q1 - q0; q0 = q1; }
        if (p.softcap_pre != 0.f) {
          // softcap: s <- tanh(s * scale / softcap); scale_log2 then holds softcap * log2(e)
#pragma unroll
          for (int i = 0; i < 64; ++i) r[i] = __float_as_uint(tanh_precise(__uint_as_float(r[i]) * p.softcap_pre));
        }
        if (cl < 63) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (i > cl) r[i] = 0xff800000u;  // -inf
        }
        if (cl_lo > 0) {
#pragma unroll
          for (int i = 0; i < 64; ++i)
            if (i < cl_lo) r[i] = 0xff800000u;
        }
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 64; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));

        if (prof) { const long long q1 = clock64(); tph1 += q1 - q0; q0 = q1; }
        // combine with the three other threads that hold parts of this row
        float* xs = xchg + xphase * 256;  // exchanges alternate between the two arrays
        xs[xi] = mx;
        t0 = prof ? clock64() : 0;
        mbar_arrive(xbar);
        ok = mbar_wait(xbar, xphase, abort_flag, p.status, ST_TIMEOUT_PEER);
        if (prof) t_b += clock64() - t0;
        ok = __all_sync(0xffffffffu, ok);
        xphase ^= 1u;
        if (!ok) break;
        mx = fmaxf(fmaxf(mx, xs[xi ^ 64]), fmaxf(xs[xi ^ 128], xs[xi ^ 192]));

        m_top = fmaxf(m_top, mx);
        float factor = 1.f;
        bool rescale = false;
        if (m_ref == -INFINITY) {
          m_ref = mx;
        } else if ((mx - m_ref) * p.scale_log2 > kRescaleThreshold) {
          factor = ex2((m_ref - mx) * p.scale_log2);
          m_ref = mx;
          l_sum *= factor;
          rescale = true;
        }
        const float ms = (m_ref == -INFINITY ? 0.f : m_ref) * p.scale_log2;
        if (prof) { const long long q1 = clock64(); tph2 += q1 - q0; q0 = q1; }

        // P = exp2(S * scale_log2 - ms), packed to 16 bit in place (masked entries are -inf -> 0)
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float a = ex2(fmaf(__uint_as_float(r[i]), p.scale_log2, -ms));
          const float b = ex2(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -ms));
          l_sum += a + b;
          r[i >> 1] = pack_half2(a, b);  // <= 2^8 by the rescale rule
        }

        if (prof) { const long long q1 = clock64(); tph3 += q1 - q0; q0 = q1; }
        // the P buffer and the O accumulators are free once PV of the previous step has completed (at the
        // first step of a tile that is the last PV of the previous tile, whose epilogue is still to come)
        if (j > 0 || have_prev) {
          t0 = prof ? clock64() : 0;
          ok = mbar_wait(ctrl + kBarPvDone, (gs - 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
          if (prof) t_c += clock64() - t0;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          tc_fence_after_sync();
        }
        if (prof) q0 = clock64();
        if (__any_sync(0xffffffffu, rescale)) {
          // this warp group rescales its half of the lane's 256 O columns
#pragma unroll 1
          for (int c4 = 0; c4 < 4; ++c4) {
            uint32_t t[32];
            const uint32_t a = lane_addr + kTmemColsO + wg * 128 + c4 * 32;
            tmem_ld32(a, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * factor);
            tmem_st32(a, t);
          }
          tmem_st_wait();
        }
        // P row segment -> shared memory, K-major 128B-swizzled [64 rows][64 keys] blocks
        {
          const uint32_t blk = sP + (half * 2 + wg) * 8192 + row * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            st_shared_v4(blk + ((c ^ (row & 7)) << 4), r[c * 4], r[c * 4 + 1], r[c * 4 + 2], r[c * 4 + 3]);
        }
        long long q2 = prof ? clock64() : 0;
        fence_proxy_async_smem();
        long long q3 = prof ? clock64() : 0;
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(leader_p_full);
        if (prof) { const long long q4 = clock64(); tph4 += q4 - q0; tph5 += q2 - q0; tph6 += q3 - q2; }
        if (j == 0 && have_prev) {
          // The previous tile's epilogue runs HERE, after this tile's first P block has been handed over:
          // the tensor pipe works on the previous tile's last PV while the first softmax step runs, and on
          // this tile's first PV (as soon as O has been read) while the stores of the epilogue drain.
          const long long te = prof ? clock64() : 0;
          epilogue(prev_b, prev_hu, prev_p0, prev_sq, prev_qoff, prev_m, prev_mt, prev_l, true);
          if (prof) t_epi += clock64() - te;
          have_prev = false;
          if (!ok) break;
        }
      }
      if (!ok) break;
      prev_b = tc.b;
      prev_hu = tc.hu;
      prev_p0 = tc.p0;
      prev_sq = tc.sq;
      prev_qoff = tc.q_off;
      prev_m = m_ref;
      prev_mt = m_top;
      prev_l = l_sum;
      have_prev = true;
    }
    if (prof && warp == 4 && lane == 0) {
      p.debug[40] = static_cast<float>(t_a);
      p.debug[41] = static_cast<float>(t_b);
      p.debug[42] = static_cast<float>(t_c);
      p.debug[43] = static_cast<float>(clock64() - t_all);
      p.debug[44] = static_cast<float>(t_epi);
      p.debug[45] = static_cast<float>(tph0);
      p.debug[46] = static_cast<float>(tph1);
      p.debug[47] = static_cast<float>(tph2);
      p.debug[48] = static_cast<float>(tph3);
      p.debug[49] = static_cast<float>(tph4);
      p.debug[50] = static_cast<float>(tph5);
      p.debug[51] = static_cast<float>(tph6);
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // give copies that may still be in flight time to land before the CTA goes away
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc<2>(tmem_base, 512);
  }
}

// V (any supported strides) -> contiguous fp16 (B,Sk,Hkv,512) / (Tk,Hkv,512); one warp per (token, head) row.
// Values beyond fp16's range saturate and |v| < 2^-14 loses bits to subnormals; attention values of ordinary
// magnitude are far from both.
__global__ void __launch_bounds__(256) splitd_fwd_vcopy_kernel(const uint16_t* v, uint16_t* v_h, int64_t n_rows,
                                                               int heads_kv, int tokens_per_batch, int64_t stride_b,
                                                               int64_t stride_s, int64_t stride_h) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int h = static_cast<int>(row % heads_kv);
  const int64_t tok = row / heads_kv;
  const int64_t b = tok / tokens_per_batch, s = tok - b * tokens_per_batch;
  store_row_half(v_h + row * kHeadDim, lane, load_row(v + b * stride_b + s * stride_s + h * stride_h, lane), 1.f);
}

size_t fwd_workspace_bytes(const splitd_params* p) {
  if (p->dtype == SPLITD_DTYPE_FP16) return 0;
  const bool varlen = p->cu_seqlens_k != nullptr;
  const int64_t tok = varlen ? p->total_k : static_cast<int64_t>(p->batch) * p->seqlen_k;
  return static_cast<size_t>((tok * p->heads_kv * kHeadDim * 2 + 255) / 256 * 256);
}

int launch_fwd(const splitd_params* p, cudaStream_t stream) {
  FwdParams fp;
  memset(&fp, 0, sizeof(fp));
  fill_geom(p, fp.g);
  const TileGeom& g = fp.g;
  CUtensorMap tm_q, tm_k, tm_v;
  if (int e = make_q_tmap(&tm_q, p->q, p, g, p->q_strides, g.pos_per_cta, "q")) return e;
  if (int e = make_kv_tmap(&tm_k, p->k, p, p->k_strides, 128, "k")) return e;
  const bool varlen_k = p->cu_seqlens_k != nullptr;
  if (p->dtype == SPLITD_DTYPE_FP16) {
    if (int e = make_kv_tmap(&tm_v, p->v, p, p->v_strides, 64, "v")) return e;
  } else {
    const size_t need = fwd_workspace_bytes(p);
    if (!p->workspace || p->workspace_bytes < need)
      return fail(SPLITD_ERR_WORKSPACE, "forward with bf16 inputs needs a workspace of %zu bytes (splitd_fwd_workspace_bytes), got %zu",
                  need, p->workspace ? p->workspace_bytes : static_cast<size_t>(0));
    if (reinterpret_cast<uintptr_t>(p->workspace) % 256 != 0 || reinterpret_cast<uintptr_t>(p->v) % 16 != 0)
      return fail(SPLITD_ERR_WORKSPACE, "workspace must be 256-byte aligned and v 16-byte aligned");
    for (int i = 0; i < 3; ++i)
      if (p->v_strides[i] % 8 != 0) return fail(SPLITD_ERR_INVALID_ARGUMENT, "v strides must be multiples of 8 elements");
    const int64_t sk = varlen_k ? p->total_k : p->seqlen_k;
    const int64_t n_rows = (varlen_k ? 1 : static_cast<int64_t>(p->batch)) * sk * p->heads_kv;
    const int64_t blocks = (n_rows + 7) / 8;
    if (blocks <= 0 || blocks > 0x7fffffffll) return fail(SPLITD_ERR_INVALID_ARGUMENT, "V copy grid out of range");
    uint16_t* v_h = static_cast<uint16_t*>(p->workspace);
    splitd_fwd_vcopy_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        static_cast<const uint16_t*>(p->v), v_h, n_rows, p->heads_kv, static_cast<int>(sk), varlen_k ? 0 : p->v_strides[0],
        p->v_strides[1], p->v_strides[2]);
    const int64_t vs[3] = {sk * p->heads_kv * kHeadDim, static_cast<int64_t>(p->heads_kv) * kHeadDim, kHeadDim};
    if (int e = make_kv_tmap(&tm_v, v_h, p, vs, 64, "v (fp16 copy)")) return e;
  }
  if (reinterpret_cast<uintptr_t>(p->o) % 16 != 0 || p->o_strides[1] % 8 != 0 || p->o_strides[2] % 8 != 0 ||
      p->o_strides[0] % 8 != 0)
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "o must be 16-byte aligned with strides that are multiples of 8 elements");
  if (reinterpret_cast<uintptr_t>(p->o_resid) % 256 != 0)
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "o_resid must be 256-byte aligned");
  fp.o = p->o;
  fp.resid_all = p->o_resid_all;
  fp.resid_flags = static_cast<uint8_t*>(p->o_resid);
  fp.resid_rows = p->o_resid ? reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(p->o_resid) + out_resid_flag_bytes(p))
                             : nullptr;
  fp.lse = p->lse;
  fp.o_stride_b = p->o_strides[0];
  fp.o_stride_s = p->o_strides[1];
  fp.o_stride_h = p->o_strides[2];
  fp.total_q = p->total_q;
  fp.scale_log2 = p->softmax_scale * kLog2e;
  fp.softcap_pre = 0.f;
  if (p->softcap > 0.f) {
    fp.softcap_pre = p->softmax_scale / p->softcap;
    fp.scale_log2 = p->softcap * kLog2e;
  }
  fp.win_left = p->local ? p->window_left : -1;
  fp.win_right = p->causal ? 0 : (p->local ? p->window_right : -1);
  fp.status = p->status_flag;
  fp.debug = p->debug;

  const bool varlen = p->cu_seqlens_q != nullptr;
  const long long pairs = varlen ? static_cast<long long>(g.row_tiles) * g.head_units
                                 : static_cast<long long>(g.row_tiles) * g.head_units * g.batch;
  if (pairs <= 0 || pairs > (1ll << 30)) return fail(SPLITD_ERR_INVALID_ARGUMENT, "forward grid out of range");
  fp.total_pairs = static_cast<int>(pairs);
  auto kern = p->dtype == SPLITD_DTYPE_FP16 ? splitd_fwd_kernel<true> : splitd_fwd_kernel<false>;
  // persistent grid: as many CTA pairs as the device can keep resident at once
  static std::atomic<int> cache[2][64];
  const int resident = resident_cluster_pairs(kern, 384, fwd::kSmemBytes, cache[p->dtype == SPLITD_DTYPE_FP16 ? 1 : 0]);
  if (resident <= 0) return fail(SPLITD_ERR_CUDA, "cudaFuncSetAttribute(forward kernel) failed");
  const long long launch_pairs = pairs < resident ? pairs : resident;
  kern<<<dim3(static_cast<unsigned>(2 * launch_pairs)), dim3(384), fwd::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, fp);
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "forward launch failed: %s", cudaGetErrorString(ce));
  return 0;
}

}  // namespace sd
