/* C ABI of libxfb200: attention forward (prefill, split-K decode, LSE merge)
 * for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only.  All tensor pointers are DEVICE pointers
 * unless a field says "host".  Strides are in ELEMENTS of the tensor's dtype.
 * Every launch goes to the stream passed by the caller (a cudaStream_t cast to
 * void*), performs no host synchronisation and reads sequence lengths, sequence
 * starts and page tables from device memory when the kernel runs, so a
 * captured CUDA graph may be replayed after those arrays were updated in place
 * (contract of the reference's callers: examples/llama_inference/generate.py:144-187).
 *
 * Return value: 0 on success, a negative XFB200_E_* code otherwise;
 * xfb200_last_error() then returns a message for the calling thread.
 *
 * The entry points replace, for this path, what the reference binds as torch
 * operators.  Its own NVIDIA kernels sit in the un-vendored `mslk` package;
 * the in-tree statement of the same boundary is the schema
 *   efficient_attention_forward_ck(query, key, value, attn_bias, seqstart_q,
 *       seqstart_k, max_seqlen_q, dropout_p, compute_logsumexp,
 *       custom_mask_type, scale, seqlen_k, window_size, block_tables, page_size)
 * (xformers/csrc/attention/attention.cpp:12-16) and
 *   efficient_attention_forward_decoder_splitk_ck
 * (xformers/csrc/attention/hip_decoder/attention_forward_splitk.cpp:94-248).
 */
#ifndef XFB200_H_
#define XFB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define XFB200_ABI_VERSION 4

#if defined(__GNUC__)
#define XFB200_API __attribute__((visibility("default")))
#else
#define XFB200_API
#endif

enum {
  XFB200_OK = 0,
  XFB200_E_INVALID = -1,     /* argument rejected by host-side validation */
  XFB200_E_UNSUPPORTED = -2, /* valid but no kernel covers it            */
  XFB200_E_CUDA = -3,        /* a CUDA runtime / driver call failed       */
  XFB200_E_DEVICE = -4       /* a kernel reported a timed-out wait        */
};

enum { XFB200_BF16 = 0, XFB200_F16 = 1, XFB200_F32 = 2 };

/* custom_mask_type of the reference boundary (attention.cpp:12-16):
 * 0 none, 1 causal aligned top-left, 2 causal aligned bottom-right.
 * 3 (prefill only): a band around the bottom-right diagonal, query i of a block
 * of mq queries and mkv keys sees key j iff
 *   i + (mkv - mq) - window_left <= j <= i + (mkv - mq) + window_right
 * (LocalAttentionFromBottomRightMask and the BlockDiagonalLocalAttention* biases,
 * xformers/ops/fmha/attn_bias.py:34-38; KAT tests/test_mem_eff_attention.py:2389-2399). */
enum { XFB200_MASK_NONE = 0, XFB200_MASK_CAUSAL_TOP_LEFT = 1, XFB200_MASK_CAUSAL_BOTTOM_RIGHT = 2, XFB200_MASK_LOCAL_BOTTOM_RIGHT = 3 };

/* kernel_path of xfb200_prefill_params: which kernel may run the call. */
enum {
  XFB200_PREFILL_AUTO = 0,        /* the fastest kernel that covers the input            */
  XFB200_PREFILL_MMA_SYNC = 1,    /* the mma.sync kernel (every head dim) */
  XFB200_PREFILL_TCGEN05 = 2,     /* fail unless a tcgen05 kernel covers the input       */
  XFB200_PREFILL_TCGEN05_CTA = 4, /* tcgen05, one CTA per block of 256 query rows        */
  XFB200_PREFILL_TCGEN05_PERSISTENT = 6 /* tcgen05, one persistent CTA per SM            */
};

enum { XFB200_KV_PLAIN = 0, XFB200_KV_INT4_ROWWISE = 1, XFB200_KV_FP8_ROWWISE = 2 };

/* [B, M, G, H, D] view of a tensor; a 4-D BMHK tensor has G = 1.  The head
 * stride of K/V may be 0 (MQA/GQA: one KV head broadcast over H query heads);
 * K/V are never expanded. */
typedef struct {
  int64_t b, m, g, h; /* last dim has stride 1 */
} xfb200_strides;

/* ---- prefill ----------------------------------------------------------------
 * O = softmax(Q K^T * scale + mask) V with optional LSE (natural log, fp32).
 * Replaces: fmha.memory_efficient_attention_forward / _forward_requires_grad
 * with a prefill operator (xformers/ops/fmha/__init__.py:40-42), schema as in
 * xformers/csrc/attention/attention.cpp:12-16.
 *
 * Dense mode  : seqstart_q == NULL; q [batch, mq, G, H, D], k/v [batch, mkv, G, H|1, D].
 * Varlen mode : seqstart_q/seqstart_k int32 [batch+1] on device, tensors carry
 *               batch 1 with sequences concatenated ("1MHK mode",
 *               hip_fmha/attention_forward_generic_ck_tiled.cpp:45-63); mq is the
 *               static bound max_seqlen_q used to size the grid.  If seqlen_k
 *               (int32 [batch]) is given, sequence b uses keys
 *               [seqstart_k[b], seqstart_k[b] + seqlen_k[b]) (padded keys).
 * kv_offset   : global index of this call's first key for the causal test;
 *               non-zero when the key axis is sharded across devices.
 */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse; /* NULL: not written.  [batch, G, H, lse_stride_h>=mq] dense; varlen: [G, H, total_q] */
  const int32_t* seqstart_q;
  const int32_t* seqstart_k;
  const int32_t* seqlen_k;
  int32_t dtype; /* XFB200_BF16 | XFB200_F16 for q, k, v, out */
  int32_t batch;
  int32_t mq;
  int32_t mkv;     /* dense: keys per batch; varlen: total key rows in the tensor */
  int32_t total_q; /* rows in q/out along dim 1 */
  int32_t groups;
  int32_t heads_per_group;
  int32_t head_dim;
  xfb200_strides q_strides, k_strides, v_strides, o_strides;
  int64_t lse_stride_b, lse_stride_g, lse_stride_h;
  int32_t mask_type;
  int32_t kv_offset;
  int32_t window_left; /* < 0: no window; else keys j >= i + shift - window_left */
  float scale;
  int32_t out_dtype; /* XFB200_BF16 | XFB200_F16 | XFB200_F32 */
  int32_t kernel_path; /* XFB200_PREFILL_*; 0 = automatic */
  /* Additive bias (a plain tensor as attn_bias, or LowerTriangularMaskWithTensorBias,
   * fmha/attn_bias.py:43; tests/test_mem_eff_attention.py:1440-1449): NULL, or
   * [batch, G, H, mq, mkv] with unit stride on the last axis and element strides
   * below (0 = broadcast), added to q k^T * scale before the mask and the softmax.
   * Dense batches only; runs on the persistent tcgen05 kernel (head dim 64 / 128) or on
   * the mma.sync kernel. */
  const void* bias;
  int32_t bias_dtype; /* XFB200_BF16 | XFB200_F16 | XFB200_F32 */
  int32_t window_right; /* XFB200_MASK_LOCAL_BOTTOM_RIGHT: keys j <= i + shift + window_right (>= 0); else ignored */
  int64_t bias_stride_b, bias_stride_g, bias_stride_h, bias_stride_m;
  /* Testing aids of the tcgen05 kernels' bounded waits; both 0 in production.
   * wait_budget_kcycles: a wait gives up after this many thousand SM clocks (0 = the default, 400000).
   * debug_flags bit 0: the first CTA does not issue its last key-tile copy, so that the wait
   * for it runs out, the kernel records a status code and returns (see xfb200_prefill_device_status). */
  int32_t wait_budget_kcycles;
  int32_t debug_flags;
  /* Two key ranges in one call (a rank of a sharded long sequence that holds two ranges of the
   * keys, stored back to back): rows [0, kv_split) of k/v start at global key kv_offset, rows
   * [kv_split, mkv) at global key kv_offset2 >= kv_offset + kv_split.  kv_split a multiple of
   * 128; 0 = one range.  Dense inputs, XFB200_MASK_CAUSAL_TOP_LEFT, no window; tcgen05 path. */
  int32_t kv_split;
  int32_t kv_offset2;
  /* The persistent tcgen05 kernel occupies every SM it is given for as long as it runs.  sm_margin > 0
   * leaves that many SMs free, for kernels of other streams that are meant to run beside it (the
   * collectives that exchange one stripe of a sharded sequence while the next one is computed). */
  int32_t sm_margin;
  int32_t reserved;
} xfb200_prefill_params;

XFB200_API int xfb200_prefill_forward(const xfb200_prefill_params* p, void* stream);

/* ---- split-K decode -----------------------------------------------------------
 * Few queries per sequence against a long KV cache that is padded
 * (sequence b at rows [b*kv_padding, b*kv_padding+seqlen_k[b])) or paged
 * (logical token t of sequence b at physical row
 *  block_tables[b*block_table_stride + t/page_size]*page_size + t%page_size),
 * in bf16/f16 or in the int4 row-wise format (one row = num_quant_groups int32
 * {scale: low fp16, shift: high fp16} followed by head_dim/8 int32 of nibbles,
 * element e of a word at bits [4e,4e+4)).
 * Replaces: fmha.triton_splitk.FwOp (xformers/ops/fmha/triton_splitk.py:18-27);
 * two-kernel structure as hip_decoder/attention_forward_splitk.cpp:58-89.
 *
 * q   [1, batch*mq, kv_heads, q_per_kv, D]   (strides m, g, h)
 * k,v [1, rows,     kv_heads, (1), D or words] (strides m, g)
 * out like q.  The key range of every sequence is cut into split_k chunks of
 * chunk_tokens(kv bound, split_k) tokens; partials go to the caller-provided
 * scratch (see xfb200_decode_scratch_bytes) and a second kernel merges them.
 */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* out;
  float* lse;         /* NULL or [kv_heads, q_per_kv, batch*mq] */
  void* scratch;      /* xfb200_decode_scratch_bytes() bytes, 256-B aligned */
  const int32_t* seqlen_k;     /* [batch]; NULL: every sequence has kv_padding keys */
  const int32_t* block_tables; /* NULL: padded cache */
  int32_t dtype;     /* of q and out (and of k/v when kv_format == PLAIN) */
  int32_t kv_format; /* XFB200_KV_PLAIN | XFB200_KV_INT4_ROWWISE | XFB200_KV_FP8_ROWWISE */
  int32_t num_quant_groups;
  int32_t batch;
  int32_t mq; /* queries per sequence (uniform) */
  int32_t kv_heads;
  int32_t q_per_kv;
  int32_t head_dim;
  int32_t kv_padding; /* padded: slot size; paged: block_table_stride*page_size */
  int32_t page_size;
  int32_t block_table_stride;
  int32_t split_k;
  int64_t q_stride_m, q_stride_g, q_stride_h;
  int64_t k_stride_m, k_stride_g;
  int64_t v_stride_m, v_stride_g;
  int64_t o_stride_m, o_stride_g, o_stride_h;
  int64_t lse_stride_g, lse_stride_h;
  int32_t mask_type; /* NONE or CAUSAL_BOTTOM_RIGHT (w.r.t. seqlen_k[b]) */
  float scale;
  int32_t out_dtype;
  /* XFB200_KV_FP8_ROWWISE: number of consecutive int32 that may be read at every (token, kv head)
   * entry of k_scale_shift / v_scale_shift, the word itself first (the reference's helper lays the
   * word out once per query head of the group, tests/utils.py:175-188).  0 or 1: only the word.
   * With 4 or more the kernel fetches the words with tiled copies.  Other formats: 0. */
  int32_t ss_words;
  /* XFB200_KV_FP8_ROWWISE only (xformers/ops/fmha/triton_splitk.py:28, InputsFp8; tests/utils.py:311-340):
   * k/v are int32 words of four e4m3 values, x = fp8 * scale + shift with one
   * (fp16 scale | fp16 shift << 16) word per token and kv head; strides in words. */
  const int32_t* k_scale_shift;
  const int32_t* v_scale_shift;
  int64_t ks_stride_m, ks_stride_g;
  int64_t vs_stride_m, vs_stride_g;
  /* Gappy caches (BlockDiagonalGappyKeysMask and its paged form, fmha/attn_bias.py:33-47): NULL, or
   * [batch] first key row of every sequence -- an absolute row of k/v for a padded cache, a row
   * inside the sequence's block table for a paged one.  kv_padding then bounds seqlen_k[b].
   * kv_rows: number of token rows of k/v (pages * page_size for a paged pool).  Required for a
   * gappy padded cache; otherwise 0 = unknown.  When given, the tiled copies are bounded by it:
   * a row past the end (a bad page-table entry) reads as zero instead of foreign memory. */
  const int32_t* kv_seqstart;
  int64_t kv_rows;
  /* Local attention (BlockDiagonalCausalLocalAttentionPaddedKeysMask,
   * PagedBlockDiagonalCausalLocalPaddedKeysMask, fmha/attn_bias.py:29,43): 0, or the number of keys a
   * query sees, the window_size keys that end at its own position (query i of the mq queries of a
   * sequence stands at key kv_len - mq + i).  Needs the bottom-right causal mask; over an int4 or fp8
   * cache, mq == 1. */
  int32_t window_size;
  int32_t reserved;
  /* Additive bias (a plain tensor as attn_bias; the reference's split-K operator takes one,
   * xformers/ops/fmha/triton_splitk.py:18-27): NULL, or [batch, kv_heads, q_per_kv, mq, keys] with unit
   * stride on the last axis and the element strides below (0 = broadcast), added to q k^T * scale
   * before the mask and the softmax.  16-bit caches in the plain layout (no sequence lengths, no
   * page table). */
  const void* bias;
  int32_t bias_dtype; /* XFB200_BF16 | XFB200_F16 | XFB200_F32 */
  int32_t reserved2;
  int64_t bias_stride_b, bias_stride_kvh, bias_stride_q, bias_stride_m;
} xfb200_decode_params;

XFB200_API size_t xfb200_decode_scratch_bytes(int32_t batch, int32_t mq, int32_t kv_heads, int32_t q_per_kv, int32_t head_dim,
                                   int32_t split_k);
XFB200_API int xfb200_decode_forward(const xfb200_decode_params* p, void* stream);

/* Split-K decode that allocates nothing.  No counterpart in the reference.
 *
 * For callers that cannot call cudaMalloc around the attention call: a serving
 * loop that must stay inside the device-memory budget it was handed at
 * start-up, a plugin inside a host application that owns the allocator, or a
 * latency-critical loop where an allocation (which may synchronise the whole
 * device) is not acceptable.  With xfb200_decode_forward such a caller would
 * have to provide the split-K scratch itself; here the library brings it.
 *
 * Same parameters and results as xfb200_decode_forward; p->scratch is ignored.
 * The per-chunk partials go to an array of XFB200_DECODE_STATIC_SCRATCH_BYTES
 * (16 MiB) that is part of the library image: every GPU that loads the library
 * holds it until the process exits.  A shape whose
 * xfb200_decode_scratch_bytes() exceeds that size is rejected with
 * XFB200_E_INVALID and a message naming both numbers: lower split_k, or use the
 * entry point above with your own scratch.  The call makes no cudaMalloc /
 * cudaFree and uses no allocating library routine.
 *
 * The first call on each device resolves the array's device address (a symbol
 * look-up with that device current, not an allocation); make that first call
 * before any stream capture.  The status word of its bounded waits is the one
 * xfb200_decode_device_status reads, also part of the library image.
 * All calls on a device share the one array, which keeps whatever the last call
 * wrote.  Nothing in it has to start at zero: every chunk that a call merges
 * has been written completely by that same call.  Two calls whose kernels may
 * overlap on the GPU (different streams or host threads) race on the array --
 * serialise them. */
#define XFB200_DECODE_STATIC_SCRATCH_BYTES (16u << 20)
XFB200_API int xfb200_decode_forward_static_scratch(const xfb200_decode_params* p, void* stream);

/* ---- merge ---------------------------------------------------------------------
 * m = max_s lse_s; w_s = exp(lse_s - m); out = sum w_s O_s / sum w_s;
 * lse = m + log sum w_s.  A partial with lse = -inf has weight 0.
 * Replaces: fmha.merge_attentions (xformers/ops/fmha/__init__.py:49,
 * xformers/ops/fmha/triton_splitk.py:29-33); arithmetic as
 * tests/test_fmha_merge_attentions.py:513-538.
 *
 * attn[s] [B, M, G, H, D] (strides b, m, g, h), lse[s] [B, G, H, M] (strides b, g, h; m has stride 1).
 * Either num_splits pointers in attn_ptrs/lse_ptrs (HOST arrays, <= XFB200_MERGE_MAX_PTRS),
 * or attn_ptrs[0]/lse_ptrs[0] plus split strides for a stacked tensor.
 */
#define XFB200_MERGE_MAX_PTRS 32
typedef struct {
  const void* const* attn_ptrs; /* host array */
  const float* const* lse_ptrs; /* host array */
  int32_t num_splits;
  int32_t stacked; /* 1: use pointer 0 and attn_stride_s / lse_stride_s */
  int64_t attn_stride_s, lse_stride_s;
  xfb200_strides attn_strides;
  int64_t lse_in_stride_b, lse_in_stride_g, lse_in_stride_h;
  void* out;
  float* lse_out; /* NULL: not written */
  xfb200_strides out_strides;
  int64_t lse_out_stride_b, lse_out_stride_g, lse_out_stride_h;
  int32_t B, M, G, H, D;
  int32_t in_dtype;  /* XFB200_F32 | XFB200_BF16 | XFB200_F16 */
  int32_t out_dtype; /* same set */
  int32_t reserved;
} xfb200_merge_params;

XFB200_API int xfb200_merge_attentions(const xfb200_merge_params* p, void* stream);

/* ------------------------------------------------------------ rope_padded
 * Rotary embeddings and KV-cache emplacement for a concatenated batch whose
 * caches are laid out as BlockDiagonalCausalWithOffsetPaddedKeysMask describes
 * (xformers/ops/rope_padded.py:16-36, kernel semantics
 * xformers/ops/_triton/rope_padded_kernels.py:13-229): for query token t of
 * sequence b (the queries of a sequence are its LAST keys),
 *   cache row = seqstart_k[b] + seqlen_k[b] - (seqstart_q[b+1] - t),
 *   position  = seqpos[t], or row - seqstart_k[b] (+ first_seqpos[b]),
 *   angle_j   = position * theta^(-2j/dim) / linear_scale   (optionally rescaled per wavelength),
 * q rows are rotated into out_q, k rows rotated into cache_k[row], v rows copied
 * into cache_v[row].  Pairs are (2j, 2j+1) when adjacents != 0, else (j, j + dim/2).
 * Strides are in elements; every row has unit stride along dim. */
typedef struct {
  const void* xq;      /* [tokens, groups, q_heads, dim] */
  const void* xk;      /* [tokens, groups, kv_heads, dim] */
  const void* xv;      /* [tokens, groups, kv_heads, dim] */
  void* out_q;         /* like xq */
  void* cache_k;       /* [cache rows, groups, kv_heads, dim], modified in place */
  void* cache_v;
  const int32_t* seqstart_q; /* [batch + 1] */
  const int32_t* seqstart_k; /* [batch + 1] */
  const int32_t* seqlen_k;   /* [batch] */
  const void* first_seqpos; /* NULL or [batch], int32 or int64 (seqpos_i64) */
  const void* seqpos;       /* NULL or [tokens], int32 or int64 (seqpos_i64) */
  int64_t seqpos_stride;    /* in elements, of whichever of the two is given */
  int32_t dtype; /* XFB200_BF16 | XFB200_F16 | XFB200_F32, of all six tensors */
  int32_t batch;
  int32_t max_q_per_seq;
  int32_t q_heads, kv_heads, groups, dim;
  int32_t adjacents;
  int32_t use_dynamic_scaling;
  int32_t internal_f64; /* angles in double precision */
  int32_t seqpos_i64;   /* first_seqpos / seqpos hold int64 */
  float theta, linear_scale;
  float dynamic_old_context_len, dynamic_scale_factor, dynamic_low_freq_factor, dynamic_high_freq_factor;
  int64_t xq_m, xq_g, xq_h;
  int64_t xk_m, xk_g, xk_h;
  int64_t xv_m, xv_g, xv_h;
  int64_t oq_m, oq_g, oq_h;
  int64_t ck_m, ck_g, ck_h;
  int64_t cv_m, cv_g, cv_h;
  /* Paged caches (an extension: the reference's rope_padded writes flat caches only).  NULL, or
   * [batch, pages per sequence]: key t of sequence b lives in row
   * block_tables[b, t / page_size] * page_size + t % page_size of cache_k / cache_v, and
   * seqstart_k is not used for addressing. */
  const int32_t* block_tables;
  int64_t block_tables_stride; /* elements between the rows of two sequences */
  int32_t page_size;
  /* 0: cache_k / cache_v have the dtype of the inputs.  2: see below.  1 (an extension as well): they are int4
   * row-wise caches of int32 rows, 1 + dim / 8 words with one quantisation group
   * (XFB200_KV_INT4_ROWWISE as the decode operator reads it); ck_* / cv_* strides count int32
   * words.  Needs bf16 / f16 inputs, dim a power of two in [32, 512], 16-byte aligned input rows. */
  int32_t cache_format;
  /* cache_format 2 (an extension as well): fp8 row-wise caches (XFB200_KV_FP8_ROWWISE): cache_k /
   * cache_v are int32 rows of dim / 4 words (strides in words, rows 8-byte aligned) and every written
   * row gets its (fp16 scale | fp16 shift << 16) word in these tensors, [cache rows, groups, kv_heads]
   * with strides in words.  shift = mean of the row, scale = max |x - shift| / 448. */
  void* k_scale_shift;
  void* v_scale_shift;
  int64_t kss_m, kss_g, kss_h;
  int64_t vss_m, vss_g, vss_h;
  /* paged caches: entries per row of block_tables.  A key position outside [0, pages_per_seq *
   * page_size) -- or, flat caches, outside the sequence's slot seqstart_k[b] .. seqstart_k[b+1] -- is
   * not written. */
  int32_t pages_per_seq;
  int32_t reserved;
} xfb200_rope_params;

XFB200_API int xfb200_rope_padded(const xfb200_rope_params* p, void* stream);


/* ---- misc ---------------------------------------------------------------------- */
XFB200_API int xfb200_abi_version(void);
XFB200_API const char* xfb200_last_error(void);
/* Every wait inside the kernels is bounded.  A kernel that gives one up records a
 * code in a status word of its device and returns; its output is then not valid.
 * These calls synchronise the given stream, store the code of the first such event
 * since the last call in *status_out (0 = none) and clear it.  They return
 * XFB200_E_DEVICE when the code is non-zero.  The words live in the library image:
 * no call of this library allocates or frees device memory for them. */
XFB200_API int xfb200_prefill_device_status(void* stream, int32_t* status_out);
XFB200_API int xfb200_decode_device_status(void* stream, int32_t* status_out);

#ifdef __cplusplus
}
#endif
#endif /* XFB200_H_ */
