/*
 * moespresso_b200 — C ABI of the B200 (sm_100a) attention hot path.
 *
 * The reference project (steadfastgaze/MoEspresso) has no FFI for this path: its
 * boundary is a set of module-level Python functions that launch Metal kernels
 * through MLX.  Each entry point below is what a binding for one of those
 * functions would call; the comment above it cites the reference function it
 * replaces (path within that project : line).
 *
 * Conventions
 *  - every pointer named in an args struct is DEVICE memory unless the comment
 *    says "host"; the library never allocates or frees user-visible memory and
 *    never synchronises the device; all work is enqueued on `stream`
 *    (a cudaStream_t passed as void*);
 *  - strides are in ELEMENTS, the innermost (feature) axis is contiguous;
 *  - return value 0 = enqueued, negative = mxb_status, with a thread-local
 *    message available from mxb_last_error();
 *  - `status` members point at one device int32 that a kernel sets non-zero
 *    when one of its bounded waits gave up (the launch still returns); may be
 *    NULL.
 */
#ifndef MOESPRESSO_B200_H
#define MOESPRESSO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MXB_ABI_VERSION 1

typedef enum {
  MXB_F32 = 0,
  MXB_F16 = 1,
  MXB_BF16 = 2,
  MXB_F8E4M3 = 3, /* FP8 E4M3FN, one byte per element */
  MXB_I8 = 4      /* int8 with one fp16 scale per row */
} mxb_dtype;

typedef enum {
  MXB_OK = 0,
  MXB_ERR_INVALID = -1,     /* contract violation (shape, dtype, alignment) */
  MXB_ERR_UNSUPPORTED = -2, /* valid request this build has no kernel for */
  MXB_ERR_WORKSPACE = -3,   /* workspace missing or too small */
  MXB_ERR_CUDA = -4         /* a CUDA runtime / driver call failed */
} mxb_status;

int mxb_abi_version(void);
const char* mxb_last_error(void);
/* Kernels this library has enqueued so far in this process (launches recorded into a CUDA graph count once,
 * when captured).  For benchmarks and tests that want to see that the device path ran. */
int64_t mxb_kernel_launches(void);
/* cudaMemcpyAsync(host -> device) on `stream`, for hosts that feed an operator's inputs from pinned memory on a
 * side stream without a CUDA binding of their own (the decode plan copies q this way while the selection runs). */
int mxb_copy_h2d_async(void* dst_device, const void* src_host, int64_t bytes, void* stream);

/* ------------------------------------------------------------------------ *
 * Indexer score.
 * Replaces  indexer_scores_tiled_live(q, weights, index_comp, *, pos0, ratio)
 *           src/moespresso/runtime/deepseek_v4/indexed_attention_kernel.py:1888-1961
 * and the decode chain  q @ pool^T -> relu -> * w -> sum_h
 *           src/moespresso/runtime/deepseek_v4/model.py:1041-1057,
 *           fused_qat_indexer_scores, indexer_score_kernel.py:354-409.
 *
 *   scores[b,t,r] = sum_h weights[b,t,h] * max(q[b,h,t,:] . keys[b][r,:], 0)
 *   ratio > 0 : scores[b,t,r] = -inf for r >= min((pos0+t+1)/ratio, rows(b))
 *   ratio == 0: no mask (decode)
 * keys of sequence b are rows [row_start[b], row_start[b] + row_count[b]) of one
 * flat [rows_total, D] table (row_start NULL: b*n_rows; row_count NULL: n_rows).
 * scores element (b,t,r) lives at
 *   scores[(row_start ? row_start[b] : 0) + b*score_stride_b + t*score_stride_t + r].
 * ------------------------------------------------------------------------ */
typedef struct {
  const void* q;        /* [B,H,T,D] via strides */
  int32_t q_dtype;      /* F32 | F16 | BF16 */
  int64_t q_stride_b, q_stride_h, q_stride_t;
  const void* keys;     /* [rows_total, D] contiguous */
  int32_t key_dtype;    /* F32 | F16 | BF16 | F8E4M3 */
  const float* weights; /* [B,T,H] contiguous */
  float* scores;
  int64_t score_stride_b, score_stride_t;
  const int64_t* row_start; /* [B] or NULL */
  const int32_t* row_count; /* [B] or NULL */
  int32_t B, T, H, D;       /* D in {64,128}; 1 <= H <= 64 */
  int64_t n_rows;           /* max rows of any sequence (host upper bound) */
  int64_t rows_total;       /* rows in the flat key table */
  int64_t pos0;
  int32_t ratio;
  int32_t flags;            /* MXB_INDEXER_* */
  int32_t* status;
  uint32_t* digit_hist;     /* NULL, or [B, 2048] counters, zero on entry: the decode scan (T == 1, ratio == 0, FP8
                               keys, 16-bit q, 8 | 16 | 32 | 64 heads; MXB_ERR_UNSUPPORTED otherwise) adds, per
                               sequence, the histogram of the top 11 bits of the selection keys of the scores it
                               writes, so that mxb_topk_select can skip its first pass (the radix select of
                               fused_decode_prep follows its scores in one launch the same way:
                               decode_attention_kernel.py:295-375) */
} mxb_indexer_scores_args;

#define MXB_INDEXER_EXACT_FP32 1 /* CUDA-core fp32 path even for 16-bit / fp8 operands */
#define MXB_INDEXER_FP8_MMA 2    /* FP8 keys fed straight to the FP8 tensor-core path (reduced-precision accumulation) */

int mxb_indexer_scores(const mxb_indexer_scores_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * Indexer QAT: Hadamard-128 + e2m1 round trip over 32-element groups, applied to
 * query heads and pool rows before the indexer score.
 * Replaces  indexer_qat_rows     src/moespresso/runtime/deepseek_v4/indexer_score_kernel.py:284-317
 *           (helper :78-134), indexer_q_qat_live
 *           src/moespresso/runtime/deepseek_v4/indexed_attention_kernel.py:1989-2027,
 *           and the composed _dsv4_indexer_qat  src/moespresso/runtime/deepseek_v4/model.py:720-749.
 *   x [n_rows, 128] f32 | f16 | bf16 (contiguous) -> out [n_rows, 128] f32.
 * ------------------------------------------------------------------------ */
typedef struct {
  const void* x;
  int32_t x_dtype;
  float* out;
  int64_t n_rows;
  int32_t width; /* must be 128 */
} mxb_indexer_qat_args;

int mxb_indexer_qat(const mxb_indexer_qat_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * Score tail of the fixed-state decode chain over per-head score rows.
 * Replaces  fused_score_tail  src/moespresso/runtime/deepseek_v4/indexer_score_kernel.py:562-615
 *           (kernel :450-490).
 *   scores [H, capacity] f32, weights_raw [H] f32 | f16 | bf16, params int32 (params[1] = valid
 *   columns) -> out [capacity] f32 = -(sum_h relu(s) * scale * (w * H^-0.5)) on the valid prefix,
 *   +inf behind it.  32 <= H <= 64.
 * ------------------------------------------------------------------------ */
typedef struct {
  const float* scores;
  const void* weights_raw;
  int32_t w_dtype;
  const int32_t* params;
  float* out;
  int32_t H;
  int64_t capacity;
  float scale;
} mxb_score_tail_args;

int mxb_score_tail(const mxb_score_tail_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * Cache-row formats.
 * mxb_fp8_kv_rows replaces  fp8_kv_prefix_rows
 *           src/moespresso/runtime/deepseek_v4/decode_attention_kernel.py:587-619 (helpers :149-176),
 *           composed _deepseek_v4_fp8_kv_roundtrip  src/moespresso/runtime/deepseek_v4/model.py:560-609:
 *   x [n_rows, 512] f32 -> out [n_rows, 512] f32, E4M3FN round trip of dims [0, 448) in 64-blocks,
 *   dims [448, 512) copied.
 * mxb_quantize_kv_int8 has no counterpart in the reference: the per-token int8 quantiser that writes
 *   the int8 + fp16-scale latent cache the sparse decode operators read.
 *   x [n_rows, width] f32 | f16 | bf16 -> q int8 [n_rows, width], scales fp16 [n_rows].
 * ------------------------------------------------------------------------ */
typedef struct {
  const float* x;
  float* out;
  int64_t n_rows;
  int32_t width; /* must be 512 */
  int32_t mode;  /* MXB_FP8KV_SERVED | MXB_FP8KV_REPLAY */
} mxb_fp8_kv_rows_args;

#define MXB_FP8KV_SERVED 0 /* the served kernel: float32 log / ceil / exp block scale, ties to the lower magnitude */
#define MXB_FP8KV_REPLAY 1 /* _fp8_kv_round of src/moespresso/correctness/deepseek_v4/compressor_diff.py:74-86:
                              exact power-of-two block scale, ties to the even code */

int mxb_fp8_kv_rows(const mxb_fp8_kv_rows_args* a, void* stream);

typedef struct {
  const void* x;
  int32_t x_dtype;
  int8_t* q;
  void* scales; /* fp16 [n_rows] */
  int64_t n_rows;
  int32_t width;
} mxb_quantize_kv_int8_args;

int mxb_quantize_kv_int8(const mxb_quantize_kv_int8_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * Affine 8-bit rows, group size 64: the format of the Qwen full-attention KV cache.
 * Replaces  mx.quantize / mx.dequantize(group_size=64, bits=8) as used on the cache and on the self chunk
 *           src/moespresso/runtime/qwen/full_attention.py:364-369 (round trip of the fresh chunk),
 *           mlx-lm QuantizedKVCache.update_and_fetch (:316, :352)
 * Per group of 64 features: bias = min, scale = (max - min) / 255, element = round((w - bias) / scale) in
 * [0, 255], w ~= element * scale + bias; four elements per uint32 (lowest byte first); scales and biases in
 * the rows' floating type.  Parity unpinned: MLX's source is not part of the reference tree.
 *   quantize:   x [n_rows, width] (row stride x_row_stride elements) -> packed, scales, biases
 *   dequantize: packed, scales, biases -> x [n_rows, width] (row stride x_row_stride; x is written)
 * ------------------------------------------------------------------------ */
typedef struct {
  const void* x;        /* rows; the OUTPUT of mxb_affine_q8_dequantize */
  int32_t x_dtype;      /* MXB_F32 | MXB_F16 | MXB_BF16 */
  int64_t x_row_stride; /* elements */
  void* packed;         /* uint32 [n_rows, width / 4] */
  void* scales;         /* [n_rows, width / 64] */
  void* biases;         /* [n_rows, width / 64] */
  int32_t sb_dtype;     /* type of scales and biases (quantize: must equal x_dtype) */
  int64_t n_rows;
  int32_t width;        /* multiple of 64 */
} mxb_affine_q8_args;

int mxb_affine_q8_quantize(const mxb_affine_q8_args* a, void* stream);
int mxb_affine_q8_dequantize(const mxb_affine_q8_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * One decode token over the affine-q8 cache, head_dim 256, split over the keys.
 * Replaces  mlx_kquant.sdpa_decode_q8(queries, *q_keys, *q_values, scale, group_size=64, bits=8, splits=128, ...)
 *           call site src/moespresso/runtime/qwen/full_attention.py:323-335 (eligibility :238-275)
 *   q [Hq, 256]; keys / values as (packed u32 [Hkv, cap, 64], scales [Hkv, cap, 4], biases [Hkv, cap, 4]) with
 *   the first P rows of every head valid and head_stride_rows = cap; q head h reads kv head h / (Hq / Hkv).
 *   Writes per-split partials o_parts [n_splits, Hq, 256] f32 and ml_parts [n_splits, Hq, 2] f32 (max in natural
 *   log units, sum); mxb_merge_partials (P = n_splits, B = T = 1) finishes.  Parity unpinned (third-party kernel).
 * ------------------------------------------------------------------------ */
typedef struct {
  const void* q;
  int32_t q_dtype;
  const void* k_packed; const void* k_scales; const void* k_biases;
  const void* v_packed; const void* v_scales; const void* v_biases;
  int32_t sb_dtype;
  int64_t head_stride_rows;
  int32_t P, Hq, Hkv, D;
  float scale;
  int32_t n_splits;
  float* o_parts;
  float* ml_parts;
} mxb_sdpa_decode_q8_args;

int mxb_sdpa_decode_q8(const mxb_sdpa_decode_q8_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * Partial rotary embedding of the last rope_dim channels (interleaved pairs), forward or inverse.
 * Replaces  apply_rope_tail  src/moespresso/runtime/deepseek_v4/attention.py:114-156 and the in-kernel
 *           rope prologue / inverse-rope epilogue of fused_decode_sdpa
 *           src/moespresso/runtime/deepseek_v4/decode_attention_kernel.py:398-422, 504-521.
 *   x, out [n_rows, width] f32 | f16 | bf16 (out may alias x); row r has position
 *   positions[r % seq_len]; inv_freq [rope_dim / 2] f64 (rope_inverse_frequencies, host side).
 * ------------------------------------------------------------------------ */
typedef struct {
  const void* x;
  void* out;
  int32_t x_dtype;
  const int64_t* positions; /* [seq_len] */
  const double* inv_freq;   /* [rope_dim / 2] */
  int64_t n_rows;
  int32_t seq_len, width, rope_dim;
  int32_t inverse;
  int32_t half_chain; /* float16 rows only: float32 angle, cos / sin and every product / sum rounded to float16,
                         as the fused decode kernels rotate (0 = float64 angles, one rounding) */
} mxb_rope_tail_args;

int mxb_rope_tail(const mxb_rope_tail_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * Top-k selection.
 * Replaces  mx.argpartition(-scores, k-1)[..., :k] + mx.sort
 *           src/moespresso/runtime/deepseek_v4/model.py:1003-1005,1057,1442-1451,
 * the radix select of fused_decode_prep
 *           src/moespresso/runtime/deepseek_v4/decode_attention_kernel.py:295-375,
 * and the NumPy contract causal_indexer_topk
 *           src/moespresso/runtime/deepseek_v4/attention.py:277-313.
 *
 * For every row: the ids of the k largest scores, ties to the LOWER id,
 * -inf / NaN never selected, -0 == +0; ids written in ASCENDING order,
 * unused slots -1.  Row i is scores[(row_start ? row_start[i] : i*row_stride) + j],
 * j < (row_count ? row_count[i] : n).
 * ------------------------------------------------------------------------ */
typedef struct {
  const float* scores;
  int64_t row_stride;
  const int64_t* row_start; /* [rows] or NULL */
  const int32_t* row_count; /* [rows] or NULL */
  int32_t* out_ids;         /* [rows, k] contiguous */
  int32_t rows;
  int64_t n;                /* max row length (host upper bound) */
  int32_t k;                /* 1 <= k <= 8192 */
  void* workspace;
  int64_t workspace_bytes;
  uint32_t* digit_hist;     /* NULL, or [rows, 2048]: the first-digit histogram of exactly the scores of each row,
                               as mxb_indexer_scores leaves it.  The selection then starts at its threshold step,
                               and the counters are zero again when the call has run (ready for the next step). */
} mxb_topk_args;

int64_t mxb_topk_workspace_bytes(int32_t rows, int64_t n, int32_t k);
int mxb_topk_select(const mxb_topk_args* a, void* stream);

/* No counterpart in the reference: the same selection for callers that must not allocate
 * device memory (a server whose memory pool is frozen after start-up, code inside another
 * allocator's callback).  `workspace` / `workspace_bytes` are ignored; the candidate
 * scratch is an 8 MiB array built into the library (2^20 entries), so rows * n must not
 * exceed 2^20.  Calls nothing that allocates.  The first call on each device looks up the
 * array's device address: make it before any stream capture.  The address is kept for the
 * life of the device's primary context: after a cudaDeviceReset in the same process the
 * library must be reloaded.  All calls share the array: calls whose kernels could overlap
 * on the GPU must be ordered (same stream). */
int mxb_topk_select_static(const mxb_topk_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * Index arithmetic of the KV-range-sharded decode step (no counterpart in the reference, which is one device):
 * the two pieces between the local kernels and the collectives, each one launch instead of a chain of
 * element-wise operations.
 * mxb_range_candidates: a rank's local top-k as (score, global id) candidates:
 *   out_scores[i] = ids[i] >= 0 ? scores[ids[i]] : -inf;  out_ids[i] = ids[i] >= 0 ? ids[i] + row_lo : -1.
 * mxb_range_local_ids: after the global selection over every rank's candidates, the rows THIS rank attends:
 *   g = pos[i] >= 0 ? cand_ids[(pos[i] / k) * cand_rank_stride + pos[i] % k] : -1;
 *   out[i] = row_lo <= g < row_lo + rows_local ? g - row_lo : -1.
 * ------------------------------------------------------------------------ */
typedef struct {
  const float* scores;    /* [rows_local] */
  const int32_t* ids;     /* [k] local ids, ascending, -1 padded */
  float* out_scores;      /* [k] */
  int32_t* out_ids;       /* [k] global ids */
  int32_t k;
  int64_t row_lo;
} mxb_range_candidates_args;

typedef struct {
  const int32_t* pos;        /* [k] positions in the rank-major list of all candidates, -1 padded */
  const int32_t* cand_ids;   /* global ids of rank r's candidates at cand_ids + r * cand_rank_stride */
  int64_t cand_rank_stride;  /* elements */
  int32_t* out;              /* [k] ids local to this rank, -1 where another rank owns the row */
  int32_t k;
  int64_t row_lo, rows_local;
} mxb_range_local_ids_args;

int mxb_range_candidates(const mxb_range_candidates_args* a, void* stream);
int mxb_range_local_ids(const mxb_range_local_ids_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * Indexed mixed (sparse) attention, decode and prefill forms.
 * Replaces  indexed_mixed_attention_decode(q, raw_kv, comp_kv, topk, sinks, *, pos0, window, ratio, raw_start)
 *           src/moespresso/runtime/deepseek_v4/indexed_attention_kernel.py:1496-1568
 *           indexed_mixed_attention_prefill / _prefill_live_f16 / _prefill_live_f32 /
 *           banded_prefill_attention_live   :2030-2108, :1571-1779, :1782-1885
 *           fused_decode_sdpa (its attention arithmetic)
 *           src/moespresso/runtime/deepseek_v4/decode_attention_kernel.py:733-786
 *
 * Token t of sequence b sits at position qpos = pos(b) + t.  It attends, per head,
 * over (1) the raw-window rows visible to qpos, (2) the rows topk[b,t,:] of the
 * compressed table in list order: id < 0 is skipped, the first id >= visible
 * ends the walk; visible = ratio ? min((qpos+1)/ratio, rows(b)) : rows(b).
 * K is the whole row (Dqk wide), V its first Dv features.  `sinks` (may be NULL)
 * adds exp(sink_h) to the denominator only.  A zero denominator yields zeros.
 *
 * partial_ml == NULL : out[b,h,t,:] = normalised attention (out_dtype F32|BF16|F16).
 * partial_ml != NULL : out must be F32 and receives sum_j exp(s_j - m) v_j;
 *                      partial_ml[b,t,h] = (m, l) as two floats, [B,T,H,2]
 *                      contiguous; the sink is NOT applied (mxb_merge_partials does).
 * ------------------------------------------------------------------------ */
typedef struct {
  const void* q;          /* [B,H,T,Dqk] via strides */
  int32_t q_dtype;        /* F32 | F16 | BF16 */
  int64_t q_stride_b, q_stride_h, q_stride_t;
  const void* comp_kv;    /* flat [comp_rows_total, Dqk] */
  int32_t kv_dtype;       /* F32 | F16 | BF16 | I8 */
  const void* comp_scales;          /* fp16 [comp_rows_total], I8 only; a row of scale 0 is a row of zeros: it adds
                                       exp(0 - m) to the denominator and nothing to the output */
  const int64_t* comp_row_start;    /* [B] or NULL: b*n_comp */
  const int32_t* comp_row_count;    /* [B] or NULL: n_comp */
  int64_t n_comp;
  const void* raw_kv;     /* [B, raw_cap, Dqk] contiguous, kv_dtype; NULL when raw_cap == 0 */
  const void* raw_scales; /* fp16 [B, raw_cap], I8 only */
  int32_t raw_cap;
  int32_t raw_start;
  const int32_t* topk;    /* [B,T,k] contiguous */
  int32_t k;
  const float* sinks;     /* [H] or NULL */
  void* out;
  int32_t out_dtype;
  int64_t out_stride_b, out_stride_h, out_stride_t;
  float* partial_ml;
  int32_t B, T, H, Dqk, Dv;
  float scale;
  int64_t pos0;            /* used when pos0_dev == NULL */
  const int64_t* pos0_dev; /* [B] or NULL */
  int32_t window, ratio;
  int32_t n_splits;        /* 0 = choose */
  int32_t flags;           /* MXB_SPARSE_* */
  void* workspace;
  int64_t workspace_bytes;
  int32_t* status;
} mxb_sparse_attn_args;

#define MXB_SPARSE_EXACT_FP32 1 /* CUDA-core fp32 kernel even where the tensor-core kernel applies */

int64_t mxb_sparse_attn_workspace_bytes(const mxb_sparse_attn_args* a);
int mxb_sparse_attn(const mxb_sparse_attn_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * Merge of (partial output, running max, running sum) triples.
 * Replaces the cross-SIMD-group (m, l) merge + sink join of fused_decode_sdpa
 *           src/moespresso/runtime/deepseek_v4/decode_attention_kernel.py:480-503
 * and is the last step of KV-range sharding across GPUs.
 *   o_parts [P, N, Dv] f32, ml_parts [P, N, 2] f32, N = B*T*H rows ordered (b,t,h).
 * ------------------------------------------------------------------------ */
typedef struct {
  const float* o_parts;
  const float* ml_parts;
  const float* sinks; /* [H] or NULL */
  void* out;
  int32_t out_dtype;
  int64_t out_stride_b, out_stride_h, out_stride_t;
  int32_t P, B, T, H, Dv;
} mxb_merge_args;

int mxb_merge_partials(const mxb_merge_args* a, void* stream);

/* ------------------------------------------------------------------------ *
 * Causal GQA flash prefill with sigmoid-gate epilogue (head_dim 256).
 * Replaces  mlx_kquant.sdpa_fa_prefill_q8(queries, *past_k, *past_v, self_k, self_v, scale, bq, bk, stage)
 *           call site src/moespresso/runtime/qwen/full_attention.py:372-382
 * plus the  out * sigmoid(gate)  of FlashPrefillD256Attention.__call__  :396-397.
 *
 *   out[i,h,:] = softmax_j(scale * q[i,h,:].k[j,h/g,:], j <= i + (Skv - S)) v[:,h/g,:]
 *                * sigmoid(gate[i,h,:])          (gate may be NULL), g = Hq/Hkv.
 * ------------------------------------------------------------------------ */
typedef struct {
  const void* q;    int64_t q_stride_s, q_stride_h;       /* [S,   Hq,  D] */
  const void* k;    int64_t k_stride_s, k_stride_h;       /* [Skv, Hkv, D] */
  const void* v;    int64_t v_stride_s, v_stride_h;       /* [Skv, Hkv, D] */
  const void* gate; int64_t gate_stride_s, gate_stride_h; /* [S,   Hq,  D] or NULL */
  void* out;        int64_t out_stride_s, out_stride_h;   /* [S,   Hq,  D] */
  int32_t dtype;    /* BF16 | F16, all five tensors */
  int32_t S, Skv, Hq, Hkv, D;
  float scale;
  void* workspace;            /* unused: the kernel needs no scratch (the size query returns 0) */
  int64_t workspace_bytes;
  int32_t* status;
} mxb_flash_prefill_args;

int64_t mxb_flash_prefill_workspace_bytes(const mxb_flash_prefill_args* a);
int mxb_flash_prefill(const mxb_flash_prefill_args* a, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOESPRESSO_B200_H */
