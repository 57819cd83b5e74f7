// Backward step 2b / 3: dQ, dK and dV as GEMMs over the bf16 P / dS tiles in the workspace
// (bwd_pds_kernel.cu), for head_dim 512 on sm_100a.
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
// is the same memory read as K-major A; dO, Q and K rows are MN-major B.
#include <cstring>

#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace sd {

namespace grad {
constexpr int kRowsPerPairOut = 256;
constexpr int kStages = 4;
constexpr int kStageBytes = 49152;  // A: 2 x 8 KB, B: 4 x 8 KB
constexpr int kOffCtrl = kStages * kStageBytes;
constexpr int kBarFull = 0;
constexpr int kBarEmpty = 8 * kStages;
constexpr int kBarAccDone = kBarEmpty + 8 * kStages;
constexpr int kTmemPtr = kBarAccDone + 8;
constexpr int kAbort = kTmemPtr + 4;
constexpr int kCtrlBytes = 256;
constexpr int kSmemBytes = kOffCtrl + kCtrlBytes;
enum { kModeDV = 0, kModeDK = 1, kModeDQ = 2 };
}  // namespace grad

struct GradLaunch {
  int n_kv_pairs;   // pairs producing dV / dK (even: dV, odd: dK)
  int n_dq_pairs;   // pairs producing dQ
  int dq_pairs_per_unit;  // packed layout: upper bound of dQ pairs per head unit; batched: per sequence
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(256, 1)
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
  const int pair_id = blockIdx.x >> 1;
  const TileGeom& g = p.g;
  const int ppp = 2 * g.pos_per_cta;  // positions per 128-row tile
  const bool folded = g.pack_g == g.group;

  // ------------------------------------------------------------------ what does this pair compute
  int mode, b = 0, sq = 0, sk = 0, q_off = 0, k_off = 0, tile_base = 0, n_row_tiles = 0;
  int kvh = 0, kt = 0;            // dK/dV: kv head, key tile (256 keys)
  int hu = 0, tp = 0;             // dQ: head unit, tile pair
  int n_stages = 0, t_min = 0, units = 1;
  if (pair_id < gl.n_kv_pairs) {
    mode = pair_id & 1;
    int idx = pair_id >> 1;
    if (g.cu_q == nullptr) {
      kt = idx % p.key_tiles;
      idx /= p.key_tiles;
      b = idx % g.batch;
      kvh = idx / g.batch;
      sq = g.seqlen_q, sk = g.seqlen_k;
      n_row_tiles = g.row_tiles;
      tile_base = b * g.row_tiles;
    } else {
      kvh = idx / p.key_tiles;
      const int r = idx - kvh * p.key_tiles;
      int acc_k = 0, acc_r = 0;
      b = -1;
      for (int i = 0; i < g.batch; ++i) {
        const int k0 = g.cu_k[i], k1 = g.cu_k[i + 1], q0 = g.cu_q[i], q1 = g.cu_q[i + 1];
        const int nkt = (k1 - k0 + 255) / 256, nrt = (q1 - q0 + ppp - 1) / ppp;
        if (r < acc_k + nkt) {
          b = i, kt = r - acc_k, sq = q1 - q0, sk = k1 - k0, q_off = q0, k_off = k0, n_row_tiles = nrt;
          break;
        }
        acc_k += nkt;
        acc_r += nrt;
      }
      if (b < 0) return;
      tile_base = acc_r;
    }
    if (kvh >= g.heads_kv) return;
    if (g.causal) {  // first row tile that can see this key tile (bottom-right aligned)
      const int x = kt * 256 - (sk - sq);
      t_min = x > 0 ? x / ppp : 0;
    }
    units = folded ? 1 : g.group;
    n_stages = units * max(n_row_tiles - t_min, 0) * 2;  // 64-row chunks
  } else {
    mode = kModeDQ;
    int idx = pair_id - gl.n_kv_pairs;
    if (g.cu_q == nullptr) {
      tp = idx % gl.dq_pairs_per_unit;
      idx /= gl.dq_pairs_per_unit;
      b = idx % g.batch;
      hu = idx / g.batch;
      sq = g.seqlen_q, sk = g.seqlen_k;
      n_row_tiles = g.row_tiles;
      tile_base = b * g.row_tiles;
      if (g.causal) tp = gl.dq_pairs_per_unit - 1 - tp;  // heaviest first
    } else {
      hu = idx / gl.dq_pairs_per_unit;
      const int r = idx - hu * gl.dq_pairs_per_unit;
      int acc_p = 0, acc_r = 0;
      b = -1;
      for (int i = 0; i < g.batch; ++i) {
        const int q0 = g.cu_q[i], q1 = g.cu_q[i + 1];
        const int nrt = (q1 - q0 + ppp - 1) / ppp, np = (nrt + 1) / 2;
        if (r < acc_p + np) {
          b = i, tp = r - acc_p, sq = q1 - q0, q_off = q0, n_row_tiles = nrt;
          k_off = g.cu_k[i];
          sk = g.cu_k[i + 1] - k_off;
          if (g.causal) tp = np - 1 - tp;
          break;
        }
        acc_p += np;
        acc_r += nrt;
      }
      if (b < 0) return;
      tile_base = acc_r;
    }
    if (hu >= g.head_units) return;
    kvh = folded ? hu : hu / g.group;
    // key extent written for this tile pair = that of its last tile, in 256-key blocks
    const int t_last = min(2 * tp + 1, n_row_tiles - 1);
    int kv_hi = sk;
    if (g.causal) kv_hi = min(kv_hi, min((t_last + 1) * ppp, sq) + sk - sq);
    n_stages = kv_hi > 0 ? ((kv_hi + 255) / 256) * 4 : 0;  // 64-key chunks
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(ctrl + kBarFull + 8 * s, 1);
      mbar_init(ctrl + kBarEmpty + 8 * s, 1);
    }
    mbar_init(ctrl + kBarAccDone, 1);
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
  // dQ: the row tile this CTA owns (clamped for loads when the last pair has a single tile)
  const int my_tile = 2 * tp + rank;
  const int my_tile_ld = min(my_tile, n_row_tiles - 1);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      uint32_t it = 0;
      auto acquire = [&](uint32_t& st, uint32_t& bar) {
        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
        ok = mbar_wait(ctrl + kBarEmpty + 8 * s, ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_LOAD);
        if (!ok) return;
        if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarFull + 8 * s, 2 * kStageBytes);
        bar = mapa_u32(ctrl + kBarFull + 8 * s, 0);
        st = sRing + s * kStageBytes;
        ++it;
      };
      if (mode != kModeDQ) {
        const CUtensorMap* tm_b = mode == kModeDK ? &tm_q : &tm_do;
        const int qb = g.cu_q ? 0 : b;
        const int key0 = kt * 256 + rank * 128;
        for (int u = 0; u < units && ok; ++u) {
          const int h = folded ? kvh : kvh * g.group + u;
          for (int t = t_min; t < n_row_tiles && ok; ++t) {
            for (int c = 0; c < 2 && ok; ++c) {
              uint32_t st = 0, bar = 0;
              acquire(st, bar);
              if (!ok) break;
              const int ws_row = (tile_base + t) * kRowsPerPair + c * kRowsPerCta;
              tma_load_3d_pair(st, &tm_ws, bar, key0, ws_row, h * 2 + mode);
              tma_load_3d_pair(st + 8192, &tm_ws, bar, key0 + 64, ws_row, h * 2 + mode);
              const int pos = q_off + t * ppp + c * g.pos_per_cta;
#pragma unroll
              for (int m = 0; m < 2; ++m) {
                const int d0 = m * 256 + rank * 128;
                tma_load_5d_pair(st + 16384 + m * 16384, tm_b, bar, d0, 0, pos, h, qb);
                tma_load_5d_pair(st + 16384 + m * 16384 + 8192, tm_b, bar, d0 + 64, 0, pos, h, qb);
              }
            }
          }
        }
      } else {
        const int kb = g.cu_k ? 0 : b;
        const int ws_row = (tile_base + my_tile_ld) * kRowsPerPair;
        for (int c = 0; c < n_stages && ok; ++c) {
          uint32_t st = 0, bar = 0;
          acquire(st, bar);
          if (!ok) break;
          tma_load_3d_pair(st, &tm_ws, bar, c * 64, ws_row, hu * 2 + 1);
          tma_load_3d_pair(st + 8192, &tm_ws, bar, c * 64, ws_row + 64, hu * 2 + 1);
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            const int d0 = m * 256 + rank * 128;
            tma_load_4d_pair(st + 16384 + m * 16384, &tm_k, bar, d0, k_off + c * 64, kvh, kb);
            tma_load_4d_pair(st + 16384 + m * 16384 + 8192, &tm_k, bar, d0 + 64, k_off + c * 64, kvh, kb);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    if (rank == 0 && lane == 0 && n_stages > 0) {
      const uint32_t idesc = make_idesc(false, mode != kModeDQ, true, 256, 256);
      const uint32_t a_step = mode != kModeDQ ? 2048u : 32u;   // 16 contraction elements further
      const uint32_t a_lbo = mode != kModeDQ ? 8192u : 16u;
      bool ok = true;
      for (int it = 0; it < n_stages && ok; ++it) {
        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
        ok = mbar_wait(ctrl + kBarFull + 8 * s, ph, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t st = sRing + s * kStageBytes;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t da = make_desc_sw128(st + k * a_step, a_lbo, 1024);
#pragma unroll
          for (int m = 0; m < 2; ++m) {
            const uint64_t db = make_desc_sw128(st + 16384 + m * 16384 + k * 2048, 8192, 1024);
            umma_ss<2>(tmem_base + m * 256, da, db, idesc, (it | k) != 0);
          }
        }
        umma_commit_pair(ctrl + kBarEmpty + 8 * s, 3);
      }
      if (ok) umma_commit_pair(ctrl + kBarAccDone, 3);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue: TMEM -> bf16 -> global
    const int q = warp & 3;
    const int L = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    bool ok = true;
    if (n_stages > 0) {
      ok = mbar_wait(ctrl + kBarAccDone, 0, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
    }
    if (ok) {
      uint16_t* drow = nullptr;
      bool store = false;
      if (mode != kModeDQ) {
        const int key = kt * 256 + rank * 128 + L;
        uint16_t* base = reinterpret_cast<uint16_t*>(mode == kModeDK ? p.dk : p.dv);
        const int64_t sb = mode == kModeDK ? p.dk_stride_b : p.dv_stride_b;
        const int64_t ss = mode == kModeDK ? p.dk_stride_s : p.dv_stride_s;
        const int64_t sh = mode == kModeDK ? p.dk_stride_h : p.dv_stride_h;
        drow = base + (g.cu_q ? 0 : b * sb) + static_cast<int64_t>(k_off + key) * ss + kvh * sh;
        store = key < sk;
      } else {
        const int pos = my_tile * ppp + L / g.pack_g;
        const int head = g.pack_g > 1 ? hu * g.pack_g + L % g.pack_g : hu;
        drow = reinterpret_cast<uint16_t*>(p.dq) + (g.cu_q ? 0 : b * p.dq_stride_b) +
               static_cast<int64_t>(q_off + pos) * p.dq_stride_s + static_cast<int64_t>(head) * p.dq_stride_h;
        store = my_tile < n_row_tiles && pos < sq;
      }
      uint32_t r[32];
#pragma unroll 1
      for (int c = 0; c < 16; ++c) {
        if (n_stages > 0) {
          tmem_ld32(lane_addr + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (store) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint32_t w[4];
#pragma unroll
            for (int t = 0; t < 4; ++t)
              w[t] = pack2<false>(__uint_as_float(r[i + 2 * t]), __uint_as_float(r[i + 2 * t + 1]));
            st_global_v4(drow + c * 32 + i, w[0], w[1], w[2], w[3]);
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

// modes: bit 0 = dK and dV, bit 1 = dQ
int launch_bwd_grad(const splitd_params* p, cudaStream_t stream, int modes) {
  BwdParams bp;
  if (int e = fill_bwd_params(p, bp)) return e;
  if (int e = check_workspace(p)) return e;
  const TileGeom& g = bp.g;
  CUtensorMap tm_ws, tm_do, tm_q, tm_k;
  {
    const uint64_t dims[3] = {(uint64_t)bp.ws_pitch, (uint64_t)bp.ws_rows, (uint64_t)(2 * g.head_units)};
    const int64_t strides[3] = {1, bp.ws_pitch, bp.ws_rows * bp.ws_pitch};
    const uint32_t box[3] = {64, 64, 1};
    if (int e = make_tmap(&tm_ws, bp.ws, 3, dims, strides, box, "workspace")) return e;
  }
  if (int e = make_q_tmap(&tm_do, p->dout, p, g, p->do_strides, g.pos_per_cta, "dout")) return e;
  if (int e = make_q_tmap(&tm_q, p->q, p, g, p->q_strides, g.pos_per_cta, "q")) return e;
  if (int e = make_kv_tmap(&tm_k, p->k, p, p->k_strides, 64, "k")) return e;
  const bool varlen = p->cu_seqlens_q != nullptr;
  GradLaunch gl;
  gl.n_kv_pairs = 0;
  gl.n_dq_pairs = 0;
  gl.dq_pairs_per_unit = varlen ? (g.row_tiles + g.batch + 1) / 2 : (g.row_tiles + 1) / 2;
  long long kv = 2ll * bp.key_tiles * g.heads_kv * (varlen ? 1 : g.batch);
  long long dq = static_cast<long long>(gl.dq_pairs_per_unit) * g.head_units * (varlen ? 1 : g.batch);
  if (!(modes & 1)) kv = 0;
  if (!(modes & 2)) dq = 0;
  const long long pairs = kv + dq;
  if (pairs <= 0 || pairs > (1ll << 30)) return fail(SPLITD_ERR_INVALID_ARGUMENT, "gradient GEMM grid out of range");
  gl.n_kv_pairs = static_cast<int>(kv);
  gl.n_dq_pairs = static_cast<int>(dq);
  cudaError_t ce =
      cudaFuncSetAttribute(splitd_bwd_grad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, grad::kSmemBytes);
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "cudaFuncSetAttribute(grad): %s", cudaGetErrorString(ce));
  splitd_bwd_grad_kernel<<<dim3(static_cast<unsigned>(2 * pairs)), dim3(256), grad::kSmemBytes, stream>>>(
      tm_ws, tm_do, tm_q, tm_k, bp, gl);
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "gradient GEMM launch failed: %s", cudaGetErrorString(ce));
  return 0;
}

int launch_bwd_dq(const splitd_params* p, cudaStream_t stream) {
  if (int e = launch_bwd_pds(p, stream)) return e;
  return launch_bwd_grad(p, stream, 2);
}
int launch_bwd_dkdv(const splitd_params* p, cudaStream_t stream) { return launch_bwd_grad(p, stream, 1); }

}  // namespace sd
