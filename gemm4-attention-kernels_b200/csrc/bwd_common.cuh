// Device helpers shared by the two backward tensor-core kernels: the power-of-two scaling of dS, chunk
// membership of row tiles, and the layout of the fp32 accumulators that travel between chunks.
#pragma once
#include "common.cuh"
#include "ptx.cuh"

namespace sd {

// P and dS are handed from the tile kernel to the gradient GEMMs as fp16 (11 significant bits; bf16 has 8, and
// its rounding of dS alone puts dQ at 1.7 - 3 x the error of a result that is rounded once). fp16 has a narrow
// exponent range, so both are scaled by powers of two, which costs no accuracy:
//   P  in (0, 1]            is stored as P * 2^14, so everything down to 2^-28 keeps full precision;
//   dS = P (dP - dpsum) scale is stored as dS * 2^e with one e per (batch or packed sequence, KV head), chosen
//      from a bound that needs no pass over dS: |dP_ij| = |dO_i . V_j| <= |dO_i| |V_j| (Cauchy-Schwarz) and
//      P <= 1 give |dS| <= (max_i |dO_i| * max_j |V_j| + max_i |dpsum_i|) * scale =: m, and e is the largest
//      integer with m * 2^e < 2^14 (fp16 overflows at 2^16). The three maxima are produced by the preprocess
//      kernel, per group, so a (batch, KV head) shard of a problem gets the same e as the whole problem.
// The B operands of the gradient GEMMs must be fp16 as well (one format per MMA): Q and K are copied as they
// are (|x| < 2^-14 loses bits to fp16's subnormals, |x| > 65504 saturates: neither happens to attention inputs
// of ordinary magnitude), dO, whose magnitude is arbitrary, as dO * 2^A with one A per group.
// The gradient kernel multiplies its accumulators by 2^-(14+A) (dV) or 2^-e (dK, dQ) before the final rounding.
constexpr int kDsBits = 14;

// Largest e with m * 2^e < 2^14 (clamped to what pow2i can represent), for m >= 0.
__device__ __forceinline__ int scale_exponent(float m) {
  const int ex = static_cast<int>(__float_as_uint(m) >> 23) & 0xff;  // m < 2^(ex - 126)
  return max(-100, min(100, kDsBits + 126 - ex));
}
// dO is copied to fp16 as dO * 2^A with A from the largest |element| of the group.
__device__ __forceinline__ int do_exponent(const uint32_t* st) { return scale_exponent(__uint_as_float(st[kStatDoMax])); }

__device__ __forceinline__ int ds_exponent(const uint32_t* st, float scale) {
  const float do2 = __uint_as_float(st[kStatDo2]), v2 = __uint_as_float(st[kStatV2]);
  const float dl = __uint_as_float(st[kStatDelta]);
  const float m = (sqrtf(do2) * sqrtf(v2) + dl) * scale * 1.001f;  // 0.1 % for the rounding of the norms themselves
  return scale_exponent(m);
}

// Row tile `rt` of the sequence whose first tile has global index `tile_base`: does it belong to the chunk?
__device__ __forceinline__ bool chunk_has_tile(const BwdParams& p, int tile_base, int rt) {
  const int gp = tile_base + (rt & ~1);
  return gp >= p.c_g0 && gp < p.c_g1;
}
// Row tiles [lo, hi) of that sequence that belong to the chunk (before clipping to the sequence).
__device__ __forceinline__ void chunk_tile_range(const BwdParams& p, int tile_base, int& lo, int& hi) {
  const int x = max(p.c_g0 - tile_base, 0), y = max(p.c_g1 - tile_base, 0);
  lo = x + (x & 1);  // smallest rt with (rt & ~1) >= x
  hi = y + (y & 1);  // one past the largest rt with (rt & ~1) < y
}
// Row of a tile inside the chunk's planes.
__device__ __forceinline__ int64_t chunk_ws_row(const BwdParams& p, int tile_base, int rt) {
  return static_cast<int64_t>(tile_base + rt - p.c_g0) * kRowsPerPair;
}

// fp32 accumulators of one (key tile, dV | dK) output tile between chunks: [tile][mode][cta rank][32-column block]
// [128 rows][32 columns], i.e. a thread's 32 consecutive columns of its TMEM lane are 128 contiguous bytes and a
// warp moves 4 KB per instruction.
constexpr int64_t kCarryFloatsPerCta = 128 * 512;
__device__ __forceinline__ float* carry_slot(const BwdParams& p, int kv_tile, int mode, int rank) {
  return p.carry + ((static_cast<int64_t>(kv_tile) * 2 + mode) * 2 + rank) * kCarryFloatsPerCta;
}

}  // namespace sd
