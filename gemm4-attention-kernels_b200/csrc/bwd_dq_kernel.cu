// Backward step 2: dQ = dS K, with P = exp2(S*scale*log2e - lse_log2), dS = P * (dP - dpsum) * scale,
// S = Q K^T, dP = dO V^T (the math of src/fmha_dq_sm90_d512.py:942-1112), for head_dim 512 on sm_100a.
//
// Query-stationary CTA pair, cta_group::2 UMMAs with M = 128 (64 packed query rows per CTA), same TMEM
// geometry as the forward kernel: dQ (64 x 512 fp32) takes columns [0,256); S and dP of one 128-key
// step take 64 columns each and are double buffered in columns [256,512). Q and dO (64 x 512 each) stay
// in shared memory for the whole tile; K and V stream through a 16 KB-stage ring: per step the K rows
// owned by this CTA for S, the V rows for dP, and the K columns owned by this CTA (all 128 keys) as
// the MN-major B operand of dQ += dS K.
//
// Besides dQ the kernel leaves every P and dS tile (bf16) in the workspace, rows in packed order, so
// that the dK/dV kernel is a pure GEMM over them and nothing is recomputed. The reference instead
// recomputes S and dP in each of four D passes of both backward kernels (3.8x the useful FLOPs).
// Steps are issued in pairs (256 keys) so the workspace is always written in 256-key blocks.
#include <cstring>

#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace sd {

namespace bdq {
constexpr int kStepKeys = 128;
constexpr int kStages = 5;
constexpr int kStageBytes = 16384;
constexpr int kOffQ = 0;
constexpr int kOffDO = 65536;
constexpr int kOffDS = 131072;
constexpr int kOffRing = kOffDS + 16384;
constexpr int kOffCtrl = kOffRing + kStages * kStageBytes;
constexpr int kBarQFull = 0;
constexpr int kBarFull = 8;
constexpr int kBarEmpty = kBarFull + 8 * kStages;
constexpr int kBarSdpFull = kBarEmpty + 8 * kStages;  // [2]
constexpr int kBarDsFull = kBarSdpFull + 16;
constexpr int kBarDqDone = kBarDsFull + 8;
constexpr int kTmemPtr = kBarDqDone + 8;
constexpr int kAbort = kTmemPtr + 4;
constexpr int kCtrlBytes = 256;
constexpr int kSmemBytes = kOffCtrl + kCtrlBytes + 1024;
constexpr int kTmemColsDQ = 0;
constexpr int kTmemColsS = 256;
}  // namespace bdq

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(256, 1)
splitd_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                     const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                     const BwdParams p) {
  using namespace bdq;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sQ = smem_base + kOffQ, sDO = smem_base + kOffDO, sDS = smem_base + kOffDS;
  const uint32_t sRing = smem_base + kOffRing, ctrl = smem_base + kOffCtrl;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffCtrl + kAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kOffCtrl + kTmemPtr);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1;
  const TileGeom& g = p.g;

  TileCoord tc;
  if (!decode_tile(g, pair_id, tc)) return;

  int kv_hi = tc.sk;
  if (g.causal) {
    const int last_pos = min(tc.p0 + 2 * g.pos_per_cta, tc.sq) - 1;
    kv_hi = min(kv_hi, last_pos + 1 + tc.sk - tc.sq);
  }
  const int n_steps = kv_hi > 0 ? 2 * ((kv_hi + 255) / 256) : 0;  // 128-key steps, issued in pairs

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(ctrl + kBarQFull, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(ctrl + kBarFull + 8 * s, 1);
      mbar_init(ctrl + kBarEmpty + 8 * s, 1);
    }
    mbar_init(ctrl + kBarSdpFull, 1);
    mbar_init(ctrl + kBarSdpFull + 8, 1);
    mbar_init(ctrl + kBarDsFull, 8);
    mbar_init(ctrl + kBarDqDone, 1);
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
  const uint32_t leader_q_full = mapa_u32(ctrl + kBarQFull, 0);
  const uint32_t leader_ds_full = mapa_u32(ctrl + kBarDsFull, 0);

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && n_steps > 0) {
      if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarQFull, 4 * 65536);
      const int qpos = tc.q_off + tc.p0 + static_cast<int>(rank) * g.pos_per_cta;
      const int qb = g.cu_q ? 0 : tc.b;
      for (int d = 0; d < 8; ++d) {
        tma_load_5d_pair(sQ + d * 8192, &tm_q, leader_q_full, d * 64, 0, qpos, tc.hu, qb);
        tma_load_5d_pair(sDO + d * 8192, &tm_do, leader_q_full, d * 64, 0, qpos, tc.hu, qb);
      }
      const int kb = g.cu_k ? 0 : tc.b;
      uint32_t it = 0;
      bool ok = true;
      auto acquire = [&]() -> uint32_t {
        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
        ok = ok && mbar_wait(ctrl + kBarEmpty + 8 * s, ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_LOAD);
        if (ok && rank == 0) mbar_arrive_expect_tx(ctrl + kBarFull + 8 * s, 2 * kStageBytes);
        ++it;
        return s;
      };
      // rows of K (or V) owned by this CTA, two 64-wide D blocks per stage
      auto load_rows = [&](const CUtensorMap* tm, int j) {
        const int key0 = tc.k_off + j * kStepKeys + static_cast<int>(rank) * 64;
        for (int c2 = 0; c2 < 4 && ok; ++c2) {
          const uint32_t s = acquire();
          if (!ok) break;
          const uint32_t bar = mapa_u32(ctrl + kBarFull + 8 * s, 0);
          tma_load_4d_pair(sRing + s * kStageBytes, tm, bar, (2 * c2) * 64, key0, tc.hkv, kb);
          tma_load_4d_pair(sRing + s * kStageBytes + 8192, tm, bar, (2 * c2 + 1) * 64, key0, tc.hkv, kb);
        }
      };
      // columns of K owned by this CTA (all keys of the step), B operand of dQ += dS K
      auto load_cols = [&](int j) {
        for (int c = 0; c < 4 && ok; ++c) {
          const int kq = c >> 1, m = c & 1;
          const uint32_t s = acquire();
          if (!ok) break;
          const uint32_t bar = mapa_u32(ctrl + kBarFull + 8 * s, 0);
          const int key0 = tc.k_off + j * kStepKeys + kq * 64;
          const int d0 = m * 256 + static_cast<int>(rank) * 128;
          tma_load_4d_pair(sRing + s * kStageBytes, &tm_k, bar, d0, key0, tc.hkv, kb);
          tma_load_4d_pair(sRing + s * kStageBytes + 8192, &tm_k, bar, d0 + 64, key0, tc.hkv, kb);
        }
      };
      load_rows(&tm_k, 0);
      load_rows(&tm_v, 0);
      for (int j = 0; j < n_steps && ok; ++j) {
        if (j + 1 < n_steps) {
          load_rows(&tm_k, j + 1);
          load_rows(&tm_v, j + 1);
        }
        load_cols(j);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA)
    if (rank == 0 && lane == 0 && n_steps > 0) {
      constexpr uint32_t idesc_s = make_idesc(false, false, false, 128, kStepKeys);
      constexpr uint32_t idesc_dq = make_idesc(false, false, true, 128, 256);
      uint32_t it = 0;
      bool ok = mbar_wait(ctrl + kBarQFull, 0, abort_flag, p.status, ST_TIMEOUT_MMA);
      tc_fence_after_sync();
      auto issue_rows = [&](uint32_t sA, uint32_t d_tmem) {
        for (int c2 = 0; c2 < 4 && ok; ++c2) {
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          ok = mbar_wait(ctrl + kBarFull + 8 * s, ph, abort_flag, p.status, ST_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int blk = k >> 2, kk = k & 3;
            const uint64_t da = make_desc_sw128(sA + (2 * c2 + blk) * 8192 + kk * 32, 16, 1024);
            const uint64_t db = make_desc_sw128(sRing + s * kStageBytes + blk * 8192 + kk * 32, 16, 1024);
            umma_ss<2>(d_tmem, da, db, idesc_s, (c2 | k) != 0);
          }
          umma_commit_pair(ctrl + kBarEmpty + 8 * s, 3);
          ++it;
        }
      };
      auto issue_sdp = [&](int j) {
        const uint32_t d_tmem = tmem_base + kTmemColsS + (j & 1) * 128;
        issue_rows(sQ, d_tmem);
        issue_rows(sDO, d_tmem + 64);
        if (ok) umma_commit_pair(ctrl + kBarSdpFull + 8 * (j & 1), 3);
      };
      auto issue_dq = [&](int j) {
        for (int c = 0; c < 4 && ok; ++c) {
          const int kq = c >> 1, m = c & 1;
          const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
          ok = mbar_wait(ctrl + kBarFull + 8 * s, ph, abort_flag, p.status, ST_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = make_desc_sw128(sDS + kq * 8192 + k * 32, 16, 1024);
            const uint64_t db = make_desc_sw128(sRing + s * kStageBytes + k * 2048, 8192, 1024);
            umma_ss<2>(tmem_base + kTmemColsDQ + m * 128, da, db, idesc_dq, (j | kq | k) != 0);
          }
          umma_commit_pair(ctrl + kBarEmpty + 8 * s, 3);
          ++it;
        }
        if (ok) umma_commit_pair(ctrl + kBarDqDone, 3);
      };
      if (ok) issue_sdp(0);
      for (int j = 0; j < n_steps && ok; ++j) {
        if (j + 1 < n_steps) issue_sdp(j + 1);
        if (!ok) break;
        ok = mbar_wait<true>(ctrl + kBarDsFull, j & 1, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after_sync();
        issue_dq(j);
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- P / dS producers + dQ epilogue
    const int q = warp & 3;
    const int L = q * 32 + lane;
    const int row = L & 63, half = L >> 6;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int pos = tc.p0 + static_cast<int>(rank) * g.pos_per_cta + row / g.pack_g;
    const int head = (g.pack_g > 1) ? tc.hu * g.pack_g + row % g.pack_g : tc.hu;
    const bool row_ok = pos < tc.sq;
    int limit = tc.sk - 1;
    if (g.causal) limit = min(limit, pos + tc.sk - tc.sq);
    if (!row_ok) limit = -1;
    float lse2 = 0.f, delta = 0.f;
    if (row_ok) {
      const int64_t idx = g.cu_q ? static_cast<int64_t>(head) * p.total_q + tc.q_off + pos
                                 : (static_cast<int64_t>(tc.b) * g.heads_q + head) * tc.sq + pos;
      lse2 = p.lse_log2[idx];
      delta = p.dpsum[idx];
    }
    const int64_t plane = p.ws_rows * p.ws_pitch;
    uint16_t* ws_p = p.ws + (static_cast<int64_t>(tc.hu) * 2) * plane +
                     (static_cast<int64_t>(tc.tile_global) * kRowsPerPair + rank * kRowsPerCta + row) * p.ws_pitch;
    uint16_t* ws_ds = ws_p + plane;

    bool ok = true;
    uint32_t r[32];
    for (int j = 0; j < n_steps && ok; ++j) {
      ok = mbar_wait(ctrl + kBarSdpFull + 8 * (j & 1), (j >> 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t s_addr = lane_addr + kTmemColsS + (j & 1) * 128;
      const int key0 = j * kStepKeys + half * 64;
      const int cl = limit - key0;
      uint32_t pk[32], dsk[32];
      float pf[32];
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        tmem_ld32(s_addr + c2 * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float pv = ex2(fmaf(__uint_as_float(r[i]), p.scale_log2, -lse2));
          pf[i] = (c2 * 32 + i > cl) ? 0.f : pv;
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) pk[c2 * 16 + (i >> 1)] = pack2<false>(pf[i], pf[i + 1]);
        tmem_ld32(s_addr + 64 + c2 * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float a = (c2 * 32 + i > cl) ? 0.f : pf[i] * (__uint_as_float(r[i]) - delta) * p.scale;
          const float b = (c2 * 32 + i + 1 > cl) ? 0.f : pf[i + 1] * (__uint_as_float(r[i + 1]) - delta) * p.scale;
          dsk[c2 * 16 + (i >> 1)] = pack2<false>(a, b);
        }
      }
      // tiles for the dK/dV kernel
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        st_global_v4(ws_p + key0 + c * 8, pk[c * 4], pk[c * 4 + 1], pk[c * 4 + 2], pk[c * 4 + 3]);
        st_global_v4(ws_ds + key0 + c * 8, dsk[c * 4], dsk[c * 4 + 1], dsk[c * 4 + 2], dsk[c * 4 + 3]);
      }
      if (j > 0) {
        ok = mbar_wait(ctrl + kBarDqDone, (j - 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      const uint32_t blk = sDS + half * 8192 + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        st_shared_v4(blk + ((c ^ (row & 7)) << 4), dsk[c * 4], dsk[c * 4 + 1], dsk[c * 4 + 2], dsk[c * 4 + 3]);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_ds_full);
    }

    if (ok && n_steps > 0) {
      ok = mbar_wait(ctrl + kBarDqDone, (n_steps - 1) & 1, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
    }
    if (ok) {
      uint16_t* drow = reinterpret_cast<uint16_t*>(p.dq) + (g.cu_q ? 0 : tc.b * p.dq_stride_b) +
                       static_cast<int64_t>(tc.q_off + pos) * p.dq_stride_s + static_cast<int64_t>(head) * p.dq_stride_h;
#pragma unroll 1
      for (int c8 = 0; c8 < 8; ++c8) {
        const int m = c8 >> 2, c4 = c8 & 3;
        if (n_steps > 0) {
          tmem_ld32(lane_addr + kTmemColsDQ + c8 * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (row_ok) {
          uint16_t* dst = drow + m * 256 + half * 128 + c4 * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int t = 0; t < 4; ++t)
              w[t] = pack2<false>(__uint_as_float(r[i + 2 * t]), __uint_as_float(r[i + 2 * t + 1]));
            st_global_v4(dst + i, w[0], w[1], w[2], w[3]);
          }
        }
      }
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

int launch_bwd_dq(const splitd_params* p, cudaStream_t stream) {
  BwdParams bp;
  if (int e = fill_bwd_params(p, bp)) return e;
  if (int e = check_workspace(p)) return e;
  const TileGeom& g = bp.g;
  CUtensorMap tm_q, tm_do, tm_k, tm_v;
  if (int e = make_q_tmap(&tm_q, p->q, p, g, p->q_strides, g.pos_per_cta, "q")) return e;
  if (int e = make_q_tmap(&tm_do, p->dout, p, g, p->do_strides, g.pos_per_cta, "dout")) return e;
  if (int e = make_kv_tmap(&tm_k, p->k, p, p->k_strides, 64, "k")) return e;
  if (int e = make_kv_tmap(&tm_v, p->v, p, p->v_strides, 64, "v")) return e;
  const bool varlen = p->cu_seqlens_q != nullptr;
  const long long pairs = varlen ? static_cast<long long>(g.row_tiles) * g.head_units
                                 : static_cast<long long>(g.row_tiles) * g.head_units * g.batch;
  if (pairs <= 0 || pairs > (1ll << 30)) return fail(SPLITD_ERR_INVALID_ARGUMENT, "dq grid out of range");
  cudaError_t ce =
      cudaFuncSetAttribute(splitd_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bdq::kSmemBytes);
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "cudaFuncSetAttribute(dq): %s", cudaGetErrorString(ce));
  splitd_bwd_dq_kernel<<<dim3(static_cast<unsigned>(2 * pairs)), dim3(256), bdq::kSmemBytes, stream>>>(
      tm_q, tm_do, tm_k, tm_v, bp);
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "dq launch failed: %s", cudaGetErrorString(ce));
  return 0;
}

}  // namespace sd
