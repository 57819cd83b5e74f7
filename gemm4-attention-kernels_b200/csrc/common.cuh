// Shared host/device definitions for the SplitD attention kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sd {

constexpr int kHeadDim = 512;
constexpr int kRowsPerCta = 64;          // packed query rows one CTA of a pair owns (UMMA M = 128 per pair)
constexpr int kRowsPerPair = 2 * kRowsPerCta;
constexpr int kChunkElems = 64;          // one 128-byte swizzle span of bf16/fp16
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
// In-kernel cycle counters (written to splitd_params::debug) exist only in builds made with -DSPLITD_PROFILE.
#ifdef SPLITD_PROFILE
constexpr bool kProfile = true;
#else
constexpr bool kProfile = false;
#endif

// Query rows are "packed": for a KV head with G query heads, row r of a tile is
// (position r / G, query head r % G), so one tile of 128 rows shares one K/V stream
// (the reference folds heads into rows the same way, src/pack_gqa.py:16-41).
// pack_g == 1 means no folding: a tile is 128 positions of a single query head.
struct TileGeom {
  int batch;
  int seqlen_q, seqlen_k;  // batched lengths; packed layout: maxima
  int heads_q, heads_kv;
  int group;               // heads_q / heads_kv
  int pack_g;              // heads folded into rows (group, or 1)
  int head_units;          // heads_kv if folded else heads_q
  int pos_per_cta;         // 64 / pack_g
  int causal;
  const int* cu_q;         // nullptr => batched
  const int* cu_k;
  int row_tiles;           // batched: tiles per sequence; packed: upper bound over all sequences
};

struct FwdParams {
  TileGeom g;
  void* o;
  uint8_t* resid_flags;  // optional low word of the output (exact output minus o, in the output dtype): one byte per
  uint16_t* resid_rows;  // row (indexed like lse) saying whether the row's low word was written, and the rows,
                         // contiguous (batch, position, head, 512) / (token, head, 512)
  int resid_all;         // 1: every row keeps its low word, not only the concentrated ones
  float* lse;
  int64_t o_stride_b, o_stride_s, o_stride_h;  // elements
  int total_q;                                 // packed: T (lse row pitch)
  float scale_log2;                            // softmax_scale * log2(e); with softcap: softcap * log2(e)
  float softcap_pre;                           // softmax_scale / softcap (0 = no softcap)
  int win_left, win_right;                     // sliding window around the diagonal, -1 = unbounded
  int total_pairs;                             // number of tile slots the persistent pairs walk over
  int* status;
  float* debug;
};

// Backward scratch ("workspace", one caller-provided buffer):
//   [0, kWsCounterBytes)           work counters of the persistent kernels
//   [kWsCounterBytes, + stats)     per (batch or packed sequence, KV head): kStatWords 32-bit words, the bit patterns of
//                                  max |dO row|^2, max |V row|^2 and max |dpsum| (they bound |dS|, see ds_exponent)
//   [dO_h, Q_h, K_h)               fp16 copies of dO (times 2^A, A per group), Q and K, contiguous (B,S,H,512) /
//                                  (T,H,512): the B operands of the gradient GEMMs, whose A operands (P, dS) are
//                                  fp16 (the two operands of one MMA must have the same format)
//   [carry)                        fp32 dK / dV accumulators that travel between chunks (only when one KV head's
//                                  rows do not fit the workspace at once)
//   [planes)                       per head unit of the CURRENT CHUNK two fp16 matrices (P * 2^14, then dS * 2^e) of
//                                  ws_rows x ws_pitch, rows in packed order (row tile * 128 + row in tile), keys of
//                                  the row's own sequence along the pitch.
// A chunk is a box (head units [c_hu0, c_hu1)) x (row tiles [c_g0, c_g1)); a row tile belongs to the chunk of the
// FIRST tile of its (even, odd) tile pair, counted over all sequences of a head unit.
struct BwdParams {
  TileGeom g;
  const float* lse;       // forward LSE (natural log)
  const float* dlse;      // may be nullptr
  float* dpsum;           // rowsum(dO*O) - dlse, same indexing as lse
  float* lse_log2;        // lse * log2(e), same indexing as lse
  const void* o;
  const uint8_t* resid_flags;   // optional low word of o as the forward left it (see FwdParams): for a row whose
  const uint16_t* resid_rows;   // flag is set, dpsum = rowsum(dO * (o + low word))
  const void* dout;
  const void* q;
  const void* k;
  const void* v;
  uint16_t* do_h;         // fp16 copies (see above)
  uint16_t* q_h;
  uint16_t* k_h;
  void* dq;
  void* dk;
  void* dv;
  int64_t o_stride_b, o_stride_s, o_stride_h;
  int64_t do_stride_b, do_stride_s, do_stride_h;
  int64_t q_stride_b, q_stride_s, q_stride_h;
  int64_t k_stride_b, k_stride_s, k_stride_h;
  int64_t v_stride_b, v_stride_s, v_stride_h;
  int64_t dq_stride_b, dq_stride_s, dq_stride_h;
  int64_t dk_stride_b, dk_stride_s, dk_stride_h;
  int64_t dv_stride_b, dv_stride_s, dv_stride_h;
  uint16_t* ws;           // planes of the current chunk
  int64_t ws_rows;        // rows per head unit in the current chunk
  int64_t ws_pitch;       // elements per row (max sequence length rounded up to 256, plus 64 of padding)
  int total_q, total_k;
  int key_tiles;          // batched: key tiles (256 keys) per sequence; packed: upper bound over all
  float scale_log2, scale;
  int* status;
  float* debug;           // optional per-role cycle counters (tests / tuning only)
  int* tile_counters;     // kWsCounterBytes at the start of the workspace
  uint32_t* stats;        // kStatWords words per (batch, KV head)
  float* carry;           // fp32 dK / dV accumulators between chunks (nullptr when no chunk splits a KV head)
  int g_end;              // row tiles per head unit (packed layout: upper bound)
  int c_hu0, c_hu1;       // chunk: head units
  int c_g0, c_g1;         // chunk: row tiles (see above)
  int c_b0, c_nb;         // batched layout: first batch / number of batches the chunk touches
  int c_tp0, c_ntp;       // batched layout: first tile pair of a sequence / number of them the chunk can touch
  int carry_mode;         // 1: dK / dV tiles may be partial in this chunk (accumulators come from / go to `carry`)
};
constexpr int kWsCounterBytes = 256;
constexpr int kCounterPds = 0, kCounterPdsDone = 8, kCounterGrad = 32, kCounterGradDone = 40;  // int offsets
constexpr int kStatWords = 4;
constexpr int kStatDo2 = 0, kStatV2 = 1, kStatDelta = 2, kStatDoMax = 3;  // kStatDoMax: max |element of dO|
constexpr int kPShift = 14;  // P is stored as P * 2^14 in fp16: P down to 2^-28 keeps all 11 significant bits

// Which tile does this CTA pair work on. Returns false when the pair has nothing to do.
struct TileCoord {
  int b, hu, hkv;
  int p0;        // first position of the pair's tile (sequence-relative)
  int sq, sk;    // this sequence's lengths
  int q_off, k_off;  // token offsets of the sequence in the packed tensors (0 when batched)
  int rt;            // row tile index inside the sequence (natural order)
  int tile_global;   // row tile index over all sequences (rows of the backward workspace / 128)
};

__device__ __forceinline__ bool decode_tile(const TileGeom& g, int pair_id, TileCoord& t) {
  const int pos_per_pair = 2 * g.pos_per_cta;
  int hu, b, rt;
  if (g.cu_q == nullptr) {
    const int bh = pair_id / g.row_tiles;
    rt = pair_id - bh * g.row_tiles;
    b = bh / g.head_units;
    hu = bh - b * g.head_units;
    if (b >= g.batch) return false;
    t.sq = g.seqlen_q;
    t.sk = g.seqlen_k;
    t.q_off = 0;
    t.k_off = 0;
    if (g.causal) rt = g.row_tiles - 1 - rt;  // heaviest tiles first
    t.tile_global = b * g.row_tiles + rt;
  } else {
    hu = pair_id / g.row_tiles;
    int idx = pair_id - hu * g.row_tiles;
    if (hu >= g.head_units) return false;
    int acc = 0;
    b = -1;
    int nt = 0;
    for (int i = 0; i < g.batch; ++i) {
      const int q0 = g.cu_q[i], q1 = g.cu_q[i + 1];
      nt = (q1 - q0 + pos_per_pair - 1) / pos_per_pair;
      if (idx < acc + nt) {
        b = i;
        t.q_off = q0;
        t.sq = q1 - q0;
        break;
      }
      acc += nt;
    }
    if (b < 0) return false;
    rt = idx - acc;
    if (g.causal) rt = nt - 1 - rt;
    t.tile_global = acc + rt;
    t.k_off = g.cu_k[b];
    t.sk = g.cu_k[b + 1] - t.k_off;
  }
  t.b = b;
  t.hu = hu;
  t.hkv = (g.pack_g == g.group) ? hu : hu / g.group;  // folded: hu is the KV head already
  t.rt = rt;
  t.p0 = rt * pos_per_pair;
  return true;
}

}  // namespace sd
