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
//
// (Measured: this 64-rows-per-CTA form issues one 64 x 256 x 16 MMA per 64 cycles, i.e. full rate.)
// Per KV step of 256 keys:  S = Q K^T (32 MMAs, K-major operands)  ->  softmax warps: row max
// (exchanged between the two threads that share a row), P = exp2(...) as bf16 into shared memory
// -> O += P V (32 MMAs, V as MN-major B operand).  S is double buffered so the tensor pipe runs
// S(j+1) while the softmax warps work on S(j).  O is only rescaled when a row max grows by more
// than 2^8 (the exact value is restored by the final 1/rowsum scaling).
//
// Warp roles (384 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only) + TMEM
// allocation, warps 4-11 softmax / epilogue: two warps per TMEM lane quarter, each thread owning 64
// of the 128 S columns of its lane, so a row of 256 keys is shared by four threads. Follows the math of the reference forward
// (src/flash_fwd_sm90_d512.py:921-1222, src/softmax.py:48-135) with a different decomposition.
#include <cstring>

#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace sd {

namespace fwd {
constexpr int kStepKeys = 256;                 // keys per KV step (UMMA N)
constexpr int kStages = 4;                     // ring stages of 32 KB
constexpr int kStageBytes = 32768;
constexpr int kQBytes = kRowsPerCta * kHeadDim * 2;     // 64 KB
constexpr int kPBytes = kRowsPerCta * kStepKeys * 2;    // 32 KB
constexpr int kOffQ = 0;
constexpr int kOffP = kOffQ + kQBytes;
constexpr int kOffRing = kOffP + kPBytes;
constexpr int kOffCtrl = kOffRing + kStages * kStageBytes;
// control block layout (bytes from kOffCtrl)
constexpr int kBarQFull = 0;
constexpr int kBarFull = 8;                        // [kStages]
constexpr int kBarEmpty = kBarFull + 8 * kStages;  // [kStages]
constexpr int kBarSFull = kBarEmpty + 8 * kStages; // [2]
constexpr int kBarPFull = kBarSFull + 16;
constexpr int kBarPvDone = kBarPFull + 8;
constexpr int kBarXchg = kBarPvDone + 8;           // [2] one per partner-warp pair
constexpr int kTmemPtr = kBarXchg + 16;
constexpr int kAbort = kTmemPtr + 4;
constexpr int kXchg = 192;                         // float [2][256]
constexpr int kCtrlBytes = kXchg + 2 * 256 * 4;
constexpr int kSmemBytes = kOffCtrl + kCtrlBytes;  // the dynamic segment is 1024-byte aligned (checked)
constexpr int kTmemColsO = 0;
constexpr int kTmemColsS = 256;
constexpr float kRescaleThreshold = 8.0f;          // log2 units
}  // namespace fwd

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
  const uint32_t sQ = smem_base + kOffQ, sP = smem_base + kOffP, sRing = smem_base + kOffRing;
  const uint32_t ctrl = smem_base + kOffCtrl;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffCtrl + kAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kOffCtrl + kTmemPtr);
  float* xchg = reinterpret_cast<float*>(smem + kOffCtrl + kXchg);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1;
  const TileGeom& g = p.g;

  // optional per-role cycle counters of one mid-grid pair (tests / tuning only)
  const bool prof = p.debug != nullptr && pair_id == static_cast<int>(gridDim.x >> 2) && cluster_ctarank() == 0;
  long long t_a = 0, t_b = 0, t_c = 0, t_all = 0;
  TileCoord tc;
  const bool has_work = decode_tile(g, pair_id, tc);  // identical in both CTAs of the pair
  if (!has_work) return;                              // uniform over the whole cluster

  // number of KV steps this tile needs
  int kv_hi = tc.sk;
  if (g.causal) {
    const int last_pos = min(tc.p0 + 2 * g.pos_per_cta, tc.sq) - 1;
    kv_hi = min(kv_hi, last_pos + 1 + tc.sk - tc.sq);
  }
  const int n_steps = kv_hi > 0 ? (kv_hi + kStepKeys - 1) / kStepKeys : 0;

  // ---------------------------------------------------------------- setup
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(ctrl + kBarQFull, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(ctrl + kBarFull + 8 * s, 1);
      mbar_init(ctrl + kBarEmpty + 8 * s, 1);
    }
    mbar_init(ctrl + kBarSFull, 1);
    mbar_init(ctrl + kBarSFull + 8, 1);
    mbar_init(ctrl + kBarPFull, 16);  // 8 softmax warps x 2 CTAs
    mbar_init(ctrl + kBarPvDone, 1);
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

  const uint32_t leader_q_full = mapa_u32(ctrl + kBarQFull, 0);
  const uint32_t leader_p_full = mapa_u32(ctrl + kBarPFull, 0);

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_steps > 0) {
      if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarQFull, 2 * kQBytes);
      const int qpos = tc.q_off + tc.p0 + static_cast<int>(rank) * g.pos_per_cta;
      const int qb = g.cu_q ? 0 : tc.b;
      for (int d = 0; d < 8; ++d)
        tma_load_5d_pair(sQ + d * 8192, &tm_q, leader_q_full, d * 64, 0, qpos, tc.hu, qb);

      const int kb = g.cu_k ? 0 : tc.b;
      uint32_t it = 0;
      bool ok = true;
      uint32_t full_bar[kStages];
#pragma unroll
      for (int s = 0; s < kStages; ++s) full_bar[s] = mapa_u32(ctrl + kBarFull + 8 * s, 0);
      auto acquire = [&](uint32_t& st, uint32_t& bar) {
        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
        const long long t0 = prof ? clock64() : 0;
        ok = ok && mbar_wait(ctrl + kBarEmpty + 8 * s, ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_LOAD);
        if (prof) t_a += clock64() - t0;
        if (ok && rank == 0) mbar_arrive_expect_tx(ctrl + kBarFull + 8 * s, 2 * kStageBytes);
        st = sRing + s * kStageBytes;
        bar = full_bar[s];
        ++it;
      };
      auto load_k = [&](int j) {  // this CTA's 128 key rows of the step, 128 of the 512 D columns per stage
        const int key0 = tc.k_off + j * kStepKeys + static_cast<int>(rank) * 128;
        for (int c = 0; c < 4 && ok; ++c) {
          uint32_t st, bar;
          acquire(st, bar);
          if (!ok) break;
          tma_load_4d_pair(st, &tm_k, bar, (2 * c) * 64, key0, tc.hkv, kb);
          tma_load_4d_pair(st + 16384, &tm_k, bar, (2 * c + 1) * 64, key0, tc.hkv, kb);
        }
      };
      auto load_v = [&](int j) {  // 64 keys per stage, this CTA's 2 x 128 V columns (both accumulators)
        for (int kq = 0; kq < 4 && ok; ++kq) {
          uint32_t st, bar;
          acquire(st, bar);
          if (!ok) break;
          const int key0 = tc.k_off + j * kStepKeys + kq * 64;
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            const int dv0 = m * 256 + static_cast<int>(rank) * 128;
            tma_load_4d_pair(st + m * 16384, &tm_v, bar, dv0, key0, tc.hkv, kb);
            tma_load_4d_pair(st + m * 16384 + 8192, &tm_v, bar, dv0 + 64, key0, tc.hkv, kb);
          }
        }
      };
      const long long tp0 = prof ? clock64() : 0;
      load_k(0);
      for (int j = 0; j < n_steps && ok; ++j) {
        if (j + 1 < n_steps) load_k(j + 1);
        load_v(j);
      }
      if (prof) {
        p.debug[100000] = static_cast<float>(t_a);
        p.debug[100001] = static_cast<float>(clock64() - tp0);
        p.debug[100002] = static_cast<float>(n_steps);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA)
    // One thread can issue a tcgen05.mma every ~45 cycles at best and each of these MMAs runs for 64, so
    // the loop is kept to a few instructions per MMA: descriptor low words are advanced by adding, the
    // high word is a constant, and one barrier wait / commit covers 8 MMAs (a 32 KB stage).
    if (rank == 0 && lane == 0 && n_steps > 0) {
      constexpr uint32_t idesc_s = make_idesc(kFp16, false, false, 128, kStepKeys);
      constexpr uint32_t idesc_pv = make_idesc(kFp16, false, true, 128, 256);
      const uint32_t q_lo = desc_lo(sQ, 16), p_lo = desc_lo(sP, 16);
      const uint32_t ring_k_lo = desc_lo(sRing, 16), ring_v_lo = desc_lo(sRing, 8192);
      uint32_t it = 0;
      t_all = prof ? clock64() : 0;
      bool ok = mbar_wait(ctrl + kBarQFull, 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      tc_fence_after_sync();
      auto issue_s = [&](int j) {
        const uint32_t d_tmem = tmem_base + kTmemColsS + (j & 1) * 128;
#pragma unroll 1
        for (int c = 0; c < 4 && ok; ++c) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          const long long t0 = prof ? clock64() : 0;
          ok = mbar_wait(ctrl + kBarFull + 8 * s, ph, abort_flag, p.status, ST_TIMEOUT_MMA);
          if (prof) t_a += clock64() - t0;
          if (!ok) break;
          const uint32_t a0 = q_lo + c * (16384 >> 4), b0 = ring_k_lo + s * (kStageBytes >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = ((k >> 2) * 8192 + (k & 3) * 32) >> 4;      // A: 8 KB per 64-wide D block
            const uint32_t offb = ((k >> 2) * 16384 + (k & 3) * 32) >> 4;    // B: 16 KB per 64-wide D block
            umma_ss<2>(d_tmem, desc_join(a0 + off), desc_join(b0 + offb), idesc_s, (c | k) != 0);
          }
          umma_commit_pair(ctrl + kBarEmpty + 8 * s, 3);
          ++it;
        }
        if (ok) umma_commit_pair(ctrl + kBarSFull + 8 * (j & 1), 3);
      };
      auto issue_pv = [&](int j) {
#pragma unroll 1
        for (int kq = 0; kq < 4 && ok; ++kq) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          const long long t0 = prof ? clock64() : 0;
          ok = mbar_wait(ctrl + kBarFull + 8 * s, ph, abort_flag, p.status, ST_TIMEOUT_MMA);
          if (prof) t_b += clock64() - t0;
          if (!ok) break;
          const uint32_t a0 = p_lo + kq * (8192 >> 4), b0 = ring_v_lo + s * (kStageBytes >> 4);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
#pragma unroll
            for (int m = 0; m < 2; ++m)
              umma_ss<2>(tmem_base + kTmemColsO + m * 128, desc_join(a0 + ((k * 32) >> 4)),
                         desc_join(b0 + ((m * 16384 + k * 2048) >> 4)), idesc_pv, (j | kq | k) != 0);
          }
          umma_commit_pair(ctrl + kBarEmpty + 8 * s, 3);
          ++it;
        }
        if (ok) umma_commit_pair(ctrl + kBarPvDone, 3);
      };
      issue_s(0);
      for (int j = 0; j < n_steps && ok; ++j) {
        if (j + 1 < n_steps) issue_s(j + 1);
        if (!ok) break;
        const long long t0 = prof ? clock64() : 0;
        ok = mbar_wait<true>(ctrl + kBarPFull, j & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (prof) t_c += clock64() - t0;
        if (!ok) break;
        tc_fence_after_sync();
        issue_pv(j);
      }
      if (prof) {
        p.debug[100004] = static_cast<float>(t_a);
        p.debug[100005] = static_cast<float>(t_b);
        p.debug[100006] = static_cast<float>(t_c);
        p.debug[100007] = static_cast<float>(clock64() - t_all);
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
    const int pos = tc.p0 + static_cast<int>(rank) * g.pos_per_cta + row / g.pack_g;
    const int head = (g.pack_g > 1) ? tc.hu * g.pack_g + row % g.pack_g : tc.hu;
    int limit = tc.sk - 1;                  // last visible key of this row
    if (g.causal) limit = min(limit, pos + tc.sk - tc.sq);
    const bool dump = (p.debug != nullptr) && pair_id == 0;

    float m_ref = -INFINITY, l_sum = 0.f;
    uint32_t xphase = 0;
    bool ok = true;
    uint32_t r[64];

    for (int j = 0; j < n_steps && ok; ++j) {
      long long t0 = prof ? clock64() : 0;
      if (j == 0) t_all = t0;
      ok = mbar_wait(ctrl + kBarSFull + 8 * (j & 1), (j >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
      if (prof) t_a += clock64() - t0;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t s_addr = lane_addr + kTmemColsS + (j & 1) * 128 + wg * 64;
      const int key0 = j * kStepKeys + half * 128 + wg * 64;  // key of this thread's column 0
      const int cl = limit - key0;                             // columns > cl are masked
      const bool masked = cl < 63;

      tmem_ld32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
      tmem_ld32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
      tmem_ld_wait();
      if (dump && j == 0) {
        float* dst = p.debug + (static_cast<int>(rank) * 128 + L) * 128 + wg * 64;
#pragma unroll
        for (int i = 0; i < 64; ++i) dst[i] = __uint_as_float(r[i]);
      }
      float mx = -INFINITY;
      if (masked) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i > cl) r[i] = 0xff800000u;  // -inf
      }
#pragma unroll
      for (int i = 0; i < 64; ++i) mx = fmaxf(mx, __uint_as_float(r[i]));

      // combine with the three other threads that hold parts of this row
      float* xs = xchg + (j & 1) * 256;
      xs[xi] = mx;
      t0 = prof ? clock64() : 0;
      mbar_arrive(xbar);
      ok = mbar_wait(xbar, xphase, abort_flag, p.status, ST_TIMEOUT_PEER);
      if (prof) t_b += clock64() - t0;
      ok = __all_sync(0xffffffffu, ok);
      xphase ^= 1u;
      if (!ok) break;
      mx = fmaxf(fmaxf(mx, xs[xi ^ 64]), fmaxf(xs[xi ^ 128], xs[xi ^ 192]));

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

      // P = exp2(S * scale_log2 - ms), packed to 16 bit in place (masked entries are -inf -> 0)
#pragma unroll
      for (int i = 0; i < 64; i += 2) {
        const float a = ex2(fmaf(__uint_as_float(r[i]), p.scale_log2, -ms));
        const float b = ex2(fmaf(__uint_as_float(r[i + 1]), p.scale_log2, -ms));
        l_sum += a + b;
        r[i >> 1] = pack2<kFp16>(a, b);
      }

      // the P buffer and the O accumulators are free once PV(j-1) has completed
      if (j > 0) {
        t0 = prof ? clock64() : 0;
        ok = mbar_wait(ctrl + kBarPvDone, (j - 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
        if (prof) t_c += clock64() - t0;
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
      }
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
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_p_full);
    }

    if (prof && warp == 4 && lane == 0) {
      p.debug[100008] = static_cast<float>(t_a);
      p.debug[100009] = static_cast<float>(t_b);
      p.debug[100010] = static_cast<float>(t_c);
      p.debug[100011] = static_cast<float>(clock64() - t_all);
    }
    // ---- epilogue
    if (ok && n_steps > 0) {
      ok = mbar_wait(ctrl + kBarPvDone, (n_steps - 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
    }
    float* xs = xchg + (n_steps & 1) * 256;
    if (ok) {
      xs[xi] = l_sum;
      mbar_arrive(xbar);
      ok = mbar_wait(xbar, xphase, abort_flag, p.status, ST_TIMEOUT_PEER);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      const float l_tot = (l_sum + xs[xi ^ 64]) + (xs[xi ^ 128] + xs[xi ^ 192]);
      const bool any = l_tot > 0.f;
      const float inv = any ? 1.f / l_tot : 0.f;
      const bool row_ok = pos < tc.sq;
      if (row_ok && half == 0 && wg == 0 && p.lse != nullptr) {
        const float ms = (m_ref == -INFINITY ? 0.f : m_ref) * p.scale_log2;
        const float lse = any ? (ms + lg2(l_tot)) * kLn2 : -INFINITY;
        const int64_t idx = g.cu_q ? static_cast<int64_t>(head) * p.total_q + tc.q_off + pos
                                   : (static_cast<int64_t>(tc.b) * g.heads_q + head) * tc.sq + pos;
        p.lse[idx] = lse;
      }
      // Epilogue stores: each thread owns one row, so a plain 16-byte store per thread would touch 32
      // different lines per warp instruction. 8 x 8 chunk transposes inside groups of 8 lanes make every
      // store instruction write 4 full 128-byte lines instead.
      uint16_t* obase = reinterpret_cast<uint16_t*>(p.o) + (g.cu_q ? 0 : tc.b * p.o_stride_b);
      const int grp_row0 = row & ~7;  // first row of this lane's group of 8
#pragma unroll 1
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t t[64];
        if (n_steps > 0) {
          tmem_ld32(lane_addr + kTmemColsO + wg * 128 + c2 * 64, *reinterpret_cast<uint32_t(*)[32]>(&t[0]));
          tmem_ld32(lane_addr + kTmemColsO + wg * 128 + c2 * 64 + 32, *reinterpret_cast<uint32_t(*)[32]>(&t[32]));
          tmem_ld_wait();
        }
        if (dump) {
          float* dst = p.debug + 32768 + (static_cast<int>(rank) * 128 + L) * 256 + wg * 128 + c2 * 64;
#pragma unroll
          for (int i = 0; i < 64; ++i) dst[i] = __uint_as_float(t[i]);
        }
        uint32_t x[32];
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float a = any ? __uint_as_float(t[i]) * inv : 0.f;
          const float b = any ? __uint_as_float(t[i + 1]) * inv : 0.f;
          x[i >> 1] = pack2<kFp16>(a, b);
        }
        transpose_chunks_8x8(x, lane);
        // now x[4r..4r+3] = 16-byte chunk (lane & 7) of row grp_row0 + r
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int rr = grp_row0 + r;
          const int pos_r = tc.p0 + static_cast<int>(rank) * g.pos_per_cta + rr / g.pack_g;
          const int head_r = (g.pack_g > 1) ? tc.hu * g.pack_g + rr % g.pack_g : tc.hu;
          if (pos_r < tc.sq) {
            uint16_t* dst = obase + static_cast<int64_t>(tc.q_off + pos_r) * p.o_stride_s +
                            static_cast<int64_t>(head_r) * p.o_stride_h + wg * 256 + half * 128 + c2 * 64 + (lane & 7) * 8;
            st_global_v4(dst, x[4 * r], x[4 * r + 1], x[4 * r + 2], x[4 * r + 3]);
          }
        }
      }
      if (dump && wg == 0) {
        float* dst = p.debug + 32768 + 65536 + (static_cast<int>(rank) * 128 + L) * 2;
        dst[0] = m_ref;
        dst[1] = l_tot;
      }
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

int launch_fwd(const splitd_params* p, cudaStream_t stream) {
  FwdParams fp;
  memset(&fp, 0, sizeof(fp));
  fill_geom(p, fp.g);
  const TileGeom& g = fp.g;
  CUtensorMap tm_q, tm_k, tm_v;
  if (int e = make_q_tmap(&tm_q, p->q, p, g, p->q_strides, g.pos_per_cta, "q")) return e;
  if (int e = make_kv_tmap(&tm_k, p->k, p, p->k_strides, 128, "k")) return e;
  if (int e = make_kv_tmap(&tm_v, p->v, p, p->v_strides, 64, "v")) return e;
  if (reinterpret_cast<uintptr_t>(p->o) % 16 != 0 || p->o_strides[1] % 8 != 0 || p->o_strides[2] % 8 != 0 ||
      p->o_strides[0] % 8 != 0)
    return fail(SPLITD_ERR_INVALID_ARGUMENT, "o must be 16-byte aligned with strides that are multiples of 8 elements");
  fp.o = p->o;
  fp.lse = p->lse;
  fp.o_stride_b = p->o_strides[0];
  fp.o_stride_s = p->o_strides[1];
  fp.o_stride_h = p->o_strides[2];
  fp.total_q = p->total_q;
  fp.scale_log2 = p->softmax_scale * kLog2e;
  fp.status = p->status_flag;
  fp.debug = p->debug;

  const bool varlen = p->cu_seqlens_q != nullptr;
  const long long pairs = varlen ? static_cast<long long>(g.row_tiles) * g.head_units
                                 : static_cast<long long>(g.row_tiles) * g.head_units * g.batch;
  if (pairs <= 0 || pairs > (1ll << 30)) return fail(SPLITD_ERR_INVALID_ARGUMENT, "forward grid out of range");
  auto kern = p->dtype == SPLITD_DTYPE_FP16 ? splitd_fwd_kernel<true> : splitd_fwd_kernel<false>;
  cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd::kSmemBytes);
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "cudaFuncSetAttribute(fwd): %s", cudaGetErrorString(ce));
  kern<<<dim3(static_cast<unsigned>(2 * pairs)), dim3(384), fwd::kSmemBytes, stream>>>(tm_q, tm_k, tm_v, fp);
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "forward launch failed: %s", cudaGetErrorString(ce));
  return 0;
}

}  // namespace sd
