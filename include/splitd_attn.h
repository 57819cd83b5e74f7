/*
 * C-ABI of the B200 (sm_100a) D=512 SplitD FlashAttention library (libsplitd_attn.so).
 *
 * These entry points are what a foreign-function binding for the reference's attention path
 * would bind. The reference (cmriat/gemm4-attention-kernels, directory splitd-flash-attn/)
 * reaches its kernels through TVM-FFI compiled functions that are called positionally from
 * src/interface.py; each function below names the call it replaces.
 *
 * Conventions
 *  - plain pointers and sizes only; every pointer is DEVICE memory owned by the caller;
 *  - the library never allocates or frees device memory, never synchronises, never throws;
 *  - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = legacy default stream);
 *  - return value: 0 on success, a negative splitd_status otherwise; a human readable message for
 *    the last failure on the calling thread is available from splitd_last_error();
 *  - head_dim is fixed to 512 for q, k and v (src/interface.py:79-87);
 *  - tensors use the reference's layouts: batched (B, S, H, 512), packed (T, H, 512) with int32
 *    cu_seqlens of B+1 entries (src/interface.py:1226-1316); the innermost (D) stride is 1 and
 *    the remaining strides are given in ELEMENTS in the params struct;
 *  - lse is fp32 (B, Hq, Sq) batched / (Hq, T) packed, natural log, -inf for rows without keys;
 *  - causal masks are bottom-right aligned: key j is visible to query i iff j <= i + Sk - Sq
 *    (tests/test_flash_fwd_splitd_sdpa.py:119-123).
 */
#ifndef SPLITD_ATTN_H_
#define SPLITD_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  SPLITD_OK = 0,
  SPLITD_ERR_INVALID_ARGUMENT = -1, /* NULL pointer, bad shape, Hq % Hkv != 0, head_dim != 512 ... */
  SPLITD_ERR_UNSUPPORTED = -2,      /* e.g. fp16 backward (src/interface.py:704-707)              */
  SPLITD_ERR_DEVICE = -3,           /* not a compute-capability 10.x device                       */
  SPLITD_ERR_CUDA = -4,             /* a CUDA runtime / driver call failed                        */
  SPLITD_ERR_WORKSPACE = -5         /* workspace missing or smaller than *_workspace_bytes()      */
} splitd_status;

enum { SPLITD_DTYPE_BF16 = 0, SPLITD_DTYPE_FP16 = 1 };

typedef struct {
  /* ---- forward operands ---- */
  const void* q; /* (B,Sq,Hq,512) or (Tq,Hq,512)   */
  const void* k; /* (B,Sk,Hkv,512) or (Tk,Hkv,512) */
  const void* v;
  void* o;    /* like q; written by forward, read by backward                */
  float* lse; /* may be NULL in forward; required by backward                */

  /* ---- backward operands (ignored by splitd_fwd) ---- */
  const void* dout;  /* like o                                                    */
  const float* dlse; /* gradient w.r.t. lse, may be NULL                          */
  void* dq;          /* like q                                                    */
  void* dk;          /* like k (already summed over the Hq/Hkv query heads)       */
  void* dv;          /* like v                                                    */
  float* dpsum;      /* fp32 scratch, splitd_bwd_rowstat_elems() elements          */
  float* lse_log2;   /* fp32 scratch, same size                                   */
  void* workspace;   /* scratch, 256-byte aligned: forward, splitd_fwd_workspace_bytes(); backward (P / dS tiles
                        and fp16 operand copies), splitd_bwd_workspace_bytes()                              */
  size_t workspace_bytes; /* how much of it the library may use                    */

  /* ---- packed (varlen) layout; both NULL selects the batched layout ---- */
  const int32_t* cu_seqlens_q; /* device, B+1 entries */
  const int32_t* cu_seqlens_k;

  /* ---- sizes ---- */
  int32_t batch;
  int32_t seqlen_q, seqlen_k; /* batched: S; packed: ignored                              */
  int32_t total_q, total_k;   /* packed: T; batched: ignored                              */
  int32_t max_seqlen_q, max_seqlen_k; /* packed: upper bounds on the sequence lengths. The backward sizes its
                                         tile rows by max_seqlen_k; a sequence with more keys than that is
                                         skipped and reported through status_flag (code 106)               */
  int32_t heads_q, heads_kv, head_dim;

  /* ---- strides in elements: {batch, sequence (token), head}; packed layout ignores [0] ---- */
  int64_t q_strides[3], k_strides[3], v_strides[3], o_strides[3];
  int64_t do_strides[3], dq_strides[3], dk_strides[3], dv_strides[3];

  float softmax_scale; /* > 0 */
  int32_t causal;      /* 0 / 1 */
  int32_t dtype;       /* SPLITD_DTYPE_* of q, k, v, o, dout, dq, dk, dv */

  /* device word, may be NULL. Every wait inside the kernels is bounded (4 s); a kernel that gives one up stores a
     positive code here with compare-and-swap against 0 and ends early, leaving its outputs incomplete:
     101 loads, 102 tensor-core issue, 103 softmax / epilogue, 104 peer CTA, 105 misaligned shared memory,
     106 a packed sequence longer than max_seqlen_k. 0 = fine. Read it after synchronising; zero it to re-arm. */
  int32_t* status_flag;

  /* reserved, must be NULL. (Builds made with -DSPLITD_PROFILE write per-role cycle counters of one CTA pair
     to the 64 floats it then points to.) */
  float* debug;

  /* ---- forward-only score modifiers (the backward rejects them, like src/interface.py:676-683) ---- */
  float softcap;        /* > 0: scores become softcap * tanh(scale * qk / softcap) before masking; 0 = off
                           (src/interface.py:446-449, src/utils.py:104-110)                              */
  int32_t local;        /* 0: no sliding window, the two fields below are ignored (so zeroed params are safe) */
  int32_t window_left;  /* >= 0: keys j < i + Sk - Sq - window_left are hidden; -1 = unbounded           */
  int32_t window_right; /* >= 0: keys j > i + Sk - Sq + window_right are hidden; -1 = unbounded          */
                        /* (sliding window of src/block_info.py:44-59; `causal` is window_right = 0)      */

  /* ---- optional low word of the output, may be NULL ---- */
  void* o_resid; /* 256-byte aligned scratch of splitd_out_resid_bytes() bytes that travels from the forward to the
                    backward of the same call. Forward: for every output row whose probability mass is concentrated
                    (largest probability > 1/16; decided per 4 rows) it receives (exact output - o), rounded to the
                    16-bit dtype, plus a byte per row saying whether it did. Backward: for those rows
                    dpsum = rowsum(dout * (o + low word)) instead of rowsum(dout * o). The rounding of o alone puts an
                    error of about |dout| * sqrt(512) * ulp(o) / 3 into dpsum; for a row that sees few keys (the first
                    rows of a causal sequence, |o| ~ |v|) that error, not the arithmetic of the kernels, decides the
                    error of dq and dk. The reference (like every backward that reads the 16-bit o,
                    src/interface.py:732-741) has it; a caller that carries o_resid from forward to backward does
                    not. The layout inside is private to the library. */
  int32_t o_resid_all; /* forward only. 0: the low word is kept for concentrated rows (above). 1: for every row. The
                          rounding of o also matters when v (or k) has a common component that is large against its
                          spread, e.g. v = 8 + N(0,1): every row then has |o| ~ 8 although no row is concentrated,
                          and dq was measured at 11.6x the SDPA-MATH error with the default, 1.2x with 1. Costs the
                          forward one more output-sized write (about 6 % at the B*S = 16384 sizes). */
} splitd_params;

/* 1 if `device` can run this library (compute capability 10.x), 0 if not, <0 on CUDA error.
 * Replaces _validate_sm90_arch (src/interface.py:123-130). */
int splitd_device_supported(int device);

/* Forward: o = softmax(q k^T * scale [+ causal mask]) v, lse = logsumexp of the scaled scores.
 * Replaces the compiled forward call `compile_cache[key](q,k,v,out,lse,scale,cu_q,cu_k,...)`
 * (src/interface.py:538-553, kernel src/flash_fwd_sm90_d512.py). bf16 or fp16.
 * With bf16 inputs the probabilities go to the tensor cores as fp16 (three more significant bits than bf16),
 * which needs v in fp16 too: the call first copies v into `workspace` (splitd_fwd_workspace_bytes(p) bytes,
 * the size of v, 256-byte aligned; `workspace_bytes` says how much is there). fp16 inputs need no workspace. */
int splitd_fwd(const splitd_params* p, void* stream);
size_t splitd_fwd_workspace_bytes(const splitd_params* p);

/* Number of fp32 elements the caller must provide in each of `dpsum` and `lse_log2`: one per (query row,
 * query head), batch * heads_q * seqlen_q or heads_q * total_q, no padding (src/interface.py:747-753 pads the
 * reference's to multiples of 64 per sequence; here tail rows are masked in the kernels instead). */
size_t splitd_bwd_rowstat_elems(const splitd_params* p);

/* Bytes of the optional `o_resid` scratch (one flag byte per output row, padded to 256, then one 16-bit row of 512
 * per output row). It is written by splitd_fwd and read by splitd_bwd / splitd_bwd_preprocess of the same problem;
 * there is no counterpart in the reference, whose backward reads the 16-bit output only (src/interface.py:732-741). */
size_t splitd_out_resid_bytes(const splitd_params* p);

/* The backward's scratch. The reference's kernels recompute S and dP in every head_dim pass and need no more
 * than the two row vectors above (src/interface.py:747-753); this library computes them once and hands the
 * P and dS tiles to the gradient GEMMs through `workspace` in fp16, 4 bytes per (query, key) pair and query head.
 * The workspace does NOT have to hold all of them: splitd_bwd cuts the problem into chunks of (KV heads, batches)
 * or, when one KV head of one batch is still too large, of row ranges whose dK/dV partial sums travel from chunk to chunk
 * in fp32, and reuses the same tile memory for every chunk. Results do not depend on the chunking, bit for bit.
 *   splitd_bwd_workspace_bytes(p)            what to allocate by default: everything at once if the tiles take at
 *                                            most 9 GiB, else up to 9 GiB of tiles plus the fixed parts (measured: whole-KV-head chunks of that
 *                                            size cost nothing, much smaller ones up to 10 %);
 *   splitd_bwd_workspace_bytes_limit(p, n)   the same with your own cap n on the tile bytes; n = 0 gives the
 *                                            smallest workspace splitd_bwd accepts, n = SIZE_MAX the size that
 *                                            holds the whole problem in one chunk.
 * Any workspace_bytes between those two extremes is accepted; more memory means fewer, larger launches. */
size_t splitd_bwd_workspace_bytes(const splitd_params* p);
size_t splitd_bwd_workspace_bytes_limit(const splitd_params* p, size_t tile_bytes_limit);

/* Backward step 1: dpsum = rowsum(o * dout) - dlse, lse_log2 = lse * log2(e).
 * Replaces `_bwd_preprocess.compile_cache[key](out,dout,dpsum,lse,lse_log2,None,cu_q,None,dlse)`
 * (src/interface.py:615-641, kernel src/flash_bwd_preprocess.py). Also clears the head of `workspace` (work
 * counters) and collects there the per-(batch, KV head) maxima that scale dS for fp16; every other backward
 * step relies on it having run first on the same workspace. */
int splitd_bwd_preprocess(const splitd_params* p, void* stream);

/* Backward step 2: dq. Replaces the dQ call `(q,k,v,dout,lse_log2,dpsum,dq,scale,cu_q,cu_k)`
 * (src/interface.py:875-886, kernel src/fmha_dq_sm90_d512.py). Also leaves the P and dS tiles of every
 * (query tile, key tile) pair in `workspace` for step 3, which is why this two-call form needs the workspace
 * of splitd_bwd_workspace_bytes_limit(p, SIZE_MAX) (SPLITD_ERR_WORKSPACE otherwise). */
int splitd_bwd_dq(const splitd_params* p, void* stream);

/* Backward step 3: dk, dv, reduced over the Hq/Hkv query heads of each KV head.
 * Replaces the dK/dV call `(q,k,v,dout,lse_log2,dpsum,dk,dv,scale,cu_q,cu_k)`
 * (src/interface.py:862-874, kernel src/fmha_dkdv_sm90_d512.py). Must follow splitd_bwd_dq on
 * the same stream with the same params. */
int splitd_bwd_dkdv(const splitd_params* p, void* stream);

/* The two launches behind steps 2 and 3, for callers that want to time or schedule them separately (no
 * counterpart in the reference, whose kernels recompute instead): splitd_bwd_tiles writes the P and dS tiles
 * (S = QK^T and dP = dO V^T on the tensor cores, as two alternating GEMM passes); splitd_bwd_grads computes dq,
 * dk and dv from them in one launch. Whole problem in one chunk, like splitd_bwd_dq. */
int splitd_bwd_tiles(const splitd_params* p, void* stream);
int splitd_bwd_grads(const splitd_params* p, void* stream);

/* The same two launches chunk by chunk, for any workspace splitd_bwd accepts: splitd_bwd_num_chunks returns how
 * many chunks the given workspace_bytes lead to (or a negative status); splitd_bwd_chunk runs `stages` (1 = tiles,
 * 2 = gradients, 3 = both) of chunk `chunk`. Chunks must run in order 0, 1, ... on one stream, tiles before
 * gradients, after splitd_bwd_preprocess: dk/dv of a KV head whose rows are spread over chunks accumulate. */
int splitd_bwd_num_chunks(const splitd_params* p);
int splitd_bwd_chunk(const splitd_params* p, int chunk, int stages, void* stream);

/* All backward steps in order on `stream` (what _flash_attn_bwd_sm90 does, src/interface.py:652-888):
 * preprocess, then tiles + gradients for every chunk. */
int splitd_bwd(const splitd_params* p, void* stream);

/* Backward (all three steps, like splitd_bwd) that allocates NOTHING and needs no scratch from the caller.
 * This entry point has no counterpart in the reference; it exists for callers that cannot call cudaMalloc:
 * a latency-critical host thread that must stay off the allocator's locks, a plugin whose host framework owns
 * all device memory and hands out only the tensors of the op, a process that was given a fixed memory budget. The scratch (dpsum, lse_log2 and
 * the P/dS workspace; those three fields of `p` are ignored) is a 17 MiB array compiled into the library
 * and resident on every GPU that loads it until the process exits.
 *  - Limits: splitd_bwd_rowstat_elems(p) <= 65536 and splitd_bwd_workspace_bytes_limit(p, SIZE_MAX) <= 16 MiB
 *    (e.g. B=1, S=512, Hq=8, Hkv=1): the problem is run in one chunk. Larger problems return SPLITD_ERR_WORKSPACE with a message that says
 *    which limit was hit; use splitd_bwd with your own buffers for those.
 *  - The first call on each device looks up the array's device address (one cudaGetSymbolAddress with that
 *    device current). Make that first call outside any stream capture.
 *  - All calls on a device share the one array and it keeps the previous call's contents. Two calls that
 *    overlap on the GPU (different streams, no dependency) race on it; order them yourself. */
int splitd_bwd_static_scratch(const splitd_params* p, void* stream);
size_t splitd_bwd_static_scratch_limit_rowstat(void);   /* 65536 floats   */
size_t splitd_bwd_static_scratch_limit_workspace(void); /* 16 MiB         */

/* Test aid, on no product path: one small CTA waits with the kernels' bounded wait on a barrier that nobody
 * arrives on, for limit_us microseconds (1 .. 100000), then stores code 104 in *status_flag (device memory)
 * and the time it waited in *waited_ns (device memory, may be NULL) and ends normally. It shows that a wait
 * that runs out leaves the kernel, the context and the GPU in working order. No counterpart in the reference. */
int splitd_wait_probe(int32_t* status_flag, unsigned int limit_us, unsigned long long* waited_ns, void* stream);

/* Message of the last failure on this thread ("" if none). */
const char* splitd_last_error(void);

/* Library version string. */
const char* splitd_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SPLITD_ATTN_H_ */
