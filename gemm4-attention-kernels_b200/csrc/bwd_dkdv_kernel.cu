// Backward step 3: dV = sum_heads P^T dO and dK = sum_heads dS^T Q for head_dim 512 on sm_100a,
// including the reduction over the Hq/Hkv query heads of each KV head (the reference loops the query
// heads inside one CTA, src/fmha_dkdv_sm90_d512.py:895-936).
//
// P and dS were left in the workspace by the dQ kernel (bf16, rows = packed query rows of a head unit,
// columns = keys), so this kernel is a plain GEMM: for 256 keys per CTA pair,
//     D[256 keys x 512] += A^T[256 keys x 64 rows] * B[64 rows x 512]
// over all packed rows that can see the key tile; A = P (for dV) or dS (for dK) read as an MN-major
// operand, B = dO or Q rows read as MN-major B. cta_group::2 UMMAs with M = 256 (128 keys per CTA,
// TMEM lane = key), N = 256 twice: the 128 x 512 fp32 accumulator fills the CTA's 512 TMEM columns.
// The GQA head reduction is simply a longer contraction: with folded heads the packed rows already
// interleave the heads; otherwise the row loop runs over each query head of the group.
// Even pairs produce dV, odd pairs dK.
#include <cstring>

#include "common.cuh"
#include "launch.cuh"
#include "ptx.cuh"

namespace sd {

namespace bkv {
constexpr int kKeysPerPair = 256;
constexpr int kStages = 4;
constexpr int kStageBytes = 49152;  // A: 2 x 8 KB, B: 4 x 8 KB
constexpr int kOffCtrl = kStages * kStageBytes;
constexpr int kBarFull = 0;
constexpr int kBarEmpty = 8 * kStages;
constexpr int kBarAccDone = kBarEmpty + 8 * kStages;
constexpr int kTmemPtr = kBarAccDone + 8;
constexpr int kAbort = kTmemPtr + 4;
constexpr int kCtrlBytes = 256;
constexpr int kSmemBytes = kOffCtrl + kCtrlBytes + 1024;
}  // namespace bkv

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(256, 1)
splitd_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_ws, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_q, const BwdParams p) {
  using namespace bkv;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t sRing = smem_base, ctrl = smem_base + kOffCtrl;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffCtrl + kAbort);
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + kOffCtrl + kTmemPtr);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1;
  const TileGeom& g = p.g;
  const int pos_per_pair = 2 * g.pos_per_cta;

  // ---- which (output, kv head, sequence, key tile)
  const int which = pair_id & 1;  // 0: dV from P and dO, 1: dK from dS and Q
  int idx = pair_id >> 1;
  int b, kt, kvh, sq, sk, q_off = 0, k_off = 0, tile_base, n_row_tiles;
  if (g.cu_q == nullptr) {
    kt = idx % p.key_tiles;
    idx /= p.key_tiles;
    b = idx % g.batch;
    kvh = idx / g.batch;
    if (kvh >= g.heads_kv) return;
    sq = g.seqlen_q;
    sk = g.seqlen_k;
    n_row_tiles = g.row_tiles;
    tile_base = b * g.row_tiles;
  } else {
    kvh = idx / p.key_tiles;
    int r = idx - kvh * p.key_tiles;
    if (kvh >= g.heads_kv) return;
    int acc_k = 0, acc_r = 0;
    b = -1;
    for (int i = 0; i < g.batch; ++i) {
      const int k0 = g.cu_k[i], k1 = g.cu_k[i + 1];
      const int q0 = g.cu_q[i], q1 = g.cu_q[i + 1];
      const int nkt = (k1 - k0 + kKeysPerPair - 1) / kKeysPerPair;
      const int nrt = (q1 - q0 + pos_per_pair - 1) / pos_per_pair;
      if (r < acc_k + nkt) {
        b = i;
        kt = r - acc_k;
        sq = q1 - q0;
        sk = k1 - k0;
        q_off = q0;
        k_off = k0;
        n_row_tiles = nrt;
        break;
      }
      acc_k += nkt;
      acc_r += nrt;
    }
    if (b < 0) return;
    tile_base = acc_r;
  }
  // first row tile that can see this key tile (causal, bottom-right aligned)
  int t_min = 0;
  if (g.causal) {
    const int x = kt * kKeysPerPair - (sk - sq);
    t_min = x > 0 ? x / pos_per_pair : 0;
  }
  const int tiles = max(n_row_tiles - t_min, 0);
  const int units = (g.pack_g == g.group) ? 1 : g.group;  // query heads looped when not folded
  const int n_stages = units * tiles * 2;                  // 64-row chunks

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(ctrl + kBarFull + 8 * s, 1);
      mbar_init(ctrl + kBarEmpty + 8 * s, 1);
    }
    mbar_init(ctrl + kBarAccDone, 1);
    fence_mbar_init();
    prefetch_tmap(&tm_ws);
    prefetch_tmap(&tm_do);
    prefetch_tmap(&tm_q);
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

  if (warp == 0) {
    if (lane == 0) {
      const CUtensorMap* tm_b = which ? &tm_q : &tm_do;
      const int qb = g.cu_q ? 0 : b;
      bool ok = true;
      uint32_t it = 0;
      for (int u = 0; u < units && ok; ++u) {
        const int hu = (g.pack_g == g.group) ? kvh : kvh * g.group + u;
        for (int t = t_min; t < n_row_tiles && ok; ++t) {
          for (int c = 0; c < 2 && ok; ++c) {
            const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
            ok = mbar_wait(ctrl + kBarEmpty + 8 * s, ph ^ 1u, abort_flag, p.status, ST_TIMEOUT_LOAD);
            if (!ok) break;
            if (rank == 0) mbar_arrive_expect_tx(ctrl + kBarFull + 8 * s, 2 * kStageBytes);
            const uint32_t bar = mapa_u32(ctrl + kBarFull + 8 * s, 0);
            const uint32_t st = sRing + s * kStageBytes;
            const int ws_row = (tile_base + t) * kRowsPerPair + c * kRowsPerCta;
            const int key0 = kt * kKeysPerPair + static_cast<int>(rank) * 128;
            tma_load_3d_pair(st, &tm_ws, bar, key0, ws_row, hu * 2 + which);
            tma_load_3d_pair(st + 8192, &tm_ws, bar, key0 + 64, ws_row, hu * 2 + which);
            const int pos = q_off + t * pos_per_pair + c * g.pos_per_cta;
#pragma unroll
            for (int m = 0; m < 2; ++m) {
              const int d0 = m * 256 + static_cast<int>(rank) * 128;
              tma_load_5d_pair(st + 16384 + m * 16384, tm_b, bar, d0, 0, pos, hu, qb);
              tma_load_5d_pair(st + 16384 + m * 16384 + 8192, tm_b, bar, d0 + 64, 0, pos, hu, qb);
            }
            ++it;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && lane == 0 && n_stages > 0) {
      constexpr uint32_t idesc = make_idesc(false, true, true, 256, 256);
      bool ok = true;
      for (int it = 0; it < n_stages && ok; ++it) {
        const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
        ok = mbar_wait(ctrl + kBarFull + 8 * s, ph, abort_flag, p.status, ST_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t st = sRing + s * kStageBytes;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t da = make_desc_sw128(st + k * 2048, 8192, 1024);
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
    const int q = warp & 3;
    const int L = q * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    const int key = kt * kKeysPerPair + static_cast<int>(rank) * 128 + L;
    bool ok = true;
    if (n_stages > 0) {
      ok = mbar_wait(ctrl + kBarAccDone, 0, abort_flag, p.status, ST_TIMEOUT_SOFTMAX);
      ok = __all_sync(0xffffffffu, ok);
      tc_fence_after_sync();
    }
    if (ok) {
      uint16_t* base = reinterpret_cast<uint16_t*>(which ? p.dk : p.dv);
      const int64_t sb = which ? p.dk_stride_b : p.dv_stride_b, ss = which ? p.dk_stride_s : p.dv_stride_s,
                    sh = which ? p.dk_stride_h : p.dv_stride_h;
      uint16_t* drow = base + (g.cu_q ? 0 : b * sb) + static_cast<int64_t>(k_off + key) * ss + kvh * sh;
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
        if (key < sk) {
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

int launch_bwd_dkdv(const splitd_params* p, cudaStream_t stream) {
  BwdParams bp;
  if (int e = fill_bwd_params(p, bp)) return e;
  if (int e = check_workspace(p)) return e;
  const TileGeom& g = bp.g;
  CUtensorMap tm_ws, tm_do, tm_q;
  {
    const uint64_t dims[3] = {(uint64_t)bp.ws_pitch, (uint64_t)bp.ws_rows, (uint64_t)(2 * g.head_units)};
    const int64_t strides[3] = {1, bp.ws_pitch, bp.ws_rows * bp.ws_pitch};
    const uint32_t box[3] = {64, 64, 1};
    if (int e = make_tmap(&tm_ws, bp.ws, 3, dims, strides, box, "workspace")) return e;
  }
  if (int e = make_q_tmap(&tm_do, p->dout, p, g, p->do_strides, g.pos_per_cta, "dout")) return e;
  if (int e = make_q_tmap(&tm_q, p->q, p, g, p->q_strides, g.pos_per_cta, "q")) return e;
  const bool varlen = p->cu_seqlens_q != nullptr;
  const long long pairs = 2ll * bp.key_tiles * g.heads_kv * (varlen ? 1 : g.batch);
  if (pairs <= 0 || pairs > (1ll << 30)) return fail(SPLITD_ERR_INVALID_ARGUMENT, "dkdv grid out of range");
  cudaError_t ce =
      cudaFuncSetAttribute(splitd_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bkv::kSmemBytes);
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "cudaFuncSetAttribute(dkdv): %s", cudaGetErrorString(ce));
  splitd_bwd_dkdv_kernel<<<dim3(static_cast<unsigned>(2 * pairs)), dim3(256), bkv::kSmemBytes, stream>>>(
      tm_ws, tm_do, tm_q, bp);
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return fail(SPLITD_ERR_CUDA, "dkdv launch failed: %s", cudaGetErrorString(ce));
  return 0;
}

}  // namespace sd
