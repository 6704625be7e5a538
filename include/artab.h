/*
 * artab.h — C ABI of libartab_b200.so: the AR-TabPFN autoregressive-sampling and
 * teacher-forced log-density hot path as hand-written sm_100a CUDA kernels.
 *
 * Conventions
 *   - Every entry point returns 0 on success or a negative ARTAB_E* code; it never
 *     throws, never synchronises the device and never allocates device memory.
 *     Buffers and workspaces are passed in by the caller, with one exception:
 *     artab_context_attention_noalloc keeps its partials in an array inside the library.
 *   - The whole-path entry points (artab_prefill, artab_decode_step, artab_decode_embedded,
 *     artab_teacher_forcing, artab_forward_masked) overlap their own kernels with programmatic
 *     dependent launch; the single-operator entry points launch plainly, because they cannot know
 *     what the caller enqueued before them.
 *   - All data pointers are device pointers unless a comment says "host".
 *   - Work is enqueued on `stream` (a cudaStream_t passed as void*).
 *   - Token rows are row-major [rows][d_model]; per-head tensors use the
 *     token-major layout [rows][n_heads][head_dim] (the reference's
 *     [B,H,Lq,Dh] transposed to put the token axis first).
 *   - dtype: ARTAB_F32 keeps q / k / v and both KV caches in fp32 and computes
 *     everything with fp32 FMA (no TF32); ARTAB_BF16 keeps q / k / v and the caches
 *     in bf16, runs the context contraction on tcgen05 tensor cores with fp32
 *     accumulation and keeps the residual stream, LayerNorm, MLP and head in fp32.
 *
 * The reference project is pure Python and has no FFI of its own; each entry
 * point below names the reference function (file:line inside the reference
 * project) whose work it takes over.
 */
#ifndef ARTAB_H_
#define ARTAB_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define ARTAB_API __attribute__((visibility("default")))
#else
#define ARTAB_API
#endif

#define ARTAB_OK 0
#define ARTAB_EINVAL (-1)     /* bad argument / unsupported shape            */
#define ARTAB_ECAPACITY (-2)  /* buffer cache or workspace too small         */
#define ARTAB_ELAUNCH (-3)    /* CUDA reported an error at launch            */
#define ARTAB_EDRIVER (-4)    /* driver entry point (tensor-map encode) missing */
#define ARTAB_ETIMEOUT (-5)   /* a bounded device-side wait gave up (artab_state.status is non-zero) */

#define ARTAB_F32 0
#define ARTAB_BF16 1

/* marker ids of Embedder (ar_tabpfn/model/model.py:36-38) */
#define ARTAB_MARK_TARGET 0
#define ARTAB_MARK_CONTEXT 1
#define ARTAB_MARK_BUFFER 2

/* ------------------------------------------------------------------------- */
/* Weights.  All fp32, all matrices stored TRANSPOSED ([in][out], row-major) so  */
/* that consecutive threads read consecutive output columns.                    */
/* ------------------------------------------------------------------------- */
typedef struct artab_layer_weights {
  const float* wf_t;    /* [D][D]   (attn_features.out_proj o attn_features.v_proj)^T:
                           feature attention over a single token reduces to this
                           product (ar_tabpfn/model/inference.py:771-773)        */
  const float* ln1_g;   /* norm1.weight [D] */
  const float* ln1_b;
  const float* wqkv_t;  /* [D][3D]  columns = [q_proj | k_proj | v_proj] of attn_rows */
  const float* wo_t;    /* [D][D]   attn_rows.out_proj^T */
  const float* ln2_g;
  const float* ln2_b;
  const float* w1_t;    /* [D][Dff]  ff.0.weight^T */
  const float* b1;      /* [Dff] */
  const float* w2_t;    /* [Dff][D]  ff.2.weight^T */
  const float* b2;      /* [D] */
  const float* ln3_g;
  const float* ln3_b;
  /* Optional bf16 copies for the tensor-core chain (NULL: the fp32 FMA chain runs).  Each is
   * the byte stream the kernel's weight ring consumes: slabs of d_model*128 bytes made of
   * [rows][64 k] blocks in the 128-byte-swizzled K-major shared-memory image, a bf16 "hi"
   * slab followed by a "lo" slab (w = hi + lo) when the matching tc_lo bit is set.
   *   tc_wo, tc_wf, tc_wqkv (q, k, v one after the other): one slab per 64-wide k-chunk, all rows;
   *   tc_w1: per 128-row output tile one 16 KB slab per k-chunk (hi part first, then lo);
 *   tc_w2: one slab per 64-wide k-chunk, all rows. */
  const void* tc_wo;
  const void* tc_w1;
  const void* tc_w2;
  const void* tc_wf;
  const void* tc_wqkv;
  int32_t tc_lo;        /* bit 0 wo, 1 w1, 2 w2, 3 wf, 4 wqkv: the matrix carries lo slabs */
  int32_t tc_reserved;
} artab_layer_weights;

typedef struct artab_model {
  int32_t d_model, n_heads, head_dim, d_ff, n_layers, n_comp, n_ar_tokens, reserved;
  const float* wx;           /* embedder.x_embed.weight[:,0] [D] */
  const float* bx;           /* embedder.x_embed.bias [D] */
  const float* wy;           /* embedder.y_embed.weight[:,0] [D] */
  const float* by;           /* embedder.y_embed.bias [D] */
  const float* marker;       /* embedder.marker_embed.weight [3][D] */
  const float* ar_tokens;    /* ar_tokens [S][D] */
  const float* lnf_g;        /* backbone.norm */
  const float* lnf_b;
  const float* wa_t;         /* head.head.0.weight^T [D][Dff] */
  const float* ba;           /* [Dff] */
  const float* wb_t;         /* head.head.2.weight^T [Dff][3K], column 3k+j, j = (mean,std,weight) */
  const float* bb;           /* [3K] */
  const float* mean_bias;    /* [K] */
  const float* std_bias;     /* [K] */
  const float* weight_bias;  /* [K] */
  const void* tc_wa;         /* head.head.0 tiled like tc_w1 (NULL: fp32 chain) */
  const void* tc_wb;         /* head.head.2 padded to 16 rows, tiled like tc_w2 */
  int32_t tc_head_lo;        /* bit 0 wa, bit 1 wb */
  int32_t tc_reserved;
  const artab_layer_weights* layers; /* HOST pointer to n_layers entries */
} artab_model;

/* ------------------------------------------------------------------------- */
/* KV-cache state and workspaces of one predictor (all device memory owned by   */
/* the caller; layout fixed at allocation, nothing is re-allocated per step).   */
/*                                                                             */
/*   k_ctx  [L][G][H][Ncp][Dh]                       context keys               */
/*   v_ctx  fp32: [L][G][H][Ncp][Dh]; bf16: [L][G][H][2*Dh][Ncp]: transposed (so  */
/*          that both tensor-core B operands are K-major) and split into a bf16  */
/*          hi part (rows 0..Dh-1) and lo part (rows Dh..2Dh-1), v = hi + lo      */
/*   kv_buf [L][B][H][T][2][Dh]   private buffer K (slot 0) and V (slot 1) of    */
/*          every stream; one stream-head's history is one contiguous span      */
/*   G = 1: one context shared by all streams ("triton_shared_context");        */
/*   G = B: one context per stream ("flex_attention" semantics).                 */
/*   Ncp = n_ctx rounded up to a multiple of 8.                                  */
/* ------------------------------------------------------------------------- */
typedef struct artab_state {
  int32_t dtype;        /* ARTAB_F32 / ARTAB_BF16 */
  int32_t n_streams;    /* B */
  int32_t n_groups;     /* G */
  int32_t n_ctx;        /* Nc */
  int32_t n_ctx_pad;    /* Ncp */
  int32_t max_buf;      /* T */
  int32_t buffer_len;   /* committed private keys per stream (host-side counter) */
  int32_t max_rows;     /* capacity of the row workspaces below */
  int32_t max_splits;   /* capacity of the partial workspaces below */
  int32_t reserved;
  void* k_ctx;
  void* v_ctx;
  void* kv_buf;
  /* max_rows must be a multiple of 128 (the tensor-core chain reads whole 128-row tiles).  In bf16
   * mode x1 and attn are library-private scratch in a lane-major tile layout; x stays row-major. */
  float* x;             /* [max_rows][D] layer input / output (residual stream) */
  float* x1;            /* [max_rows][D] post-norm1 activations */
  float* attn;          /* [max_rows][D] merged attention output */
  void* q;              /* [max_rows][H][Dh] queries, cache dtype */
  float* o_part;        /* [max_splits][max_rows][H][Dh] context partial outputs; between the attention
                         * stages the tensor-core dense chain uses slots 0-5 as scratch for its CTA
                         * pairs (max_splits < 6: one CTA per row tile) */
  float* lse_part;      /* [max_splits][max_rows][H] natural-log LSE of each partial */
  int32_t* status;      /* device word: 0, or the code of a bounded wait that gave up */
} artab_state;

/* --------------------------- whole-path entry points ---------------------- */

/* Context prefill: embeds G x n_ctx labelled rows, runs every layer with dense
 * (non-causal) self-attention and writes the context K/V of every layer into
 * st->k_ctx / st->v_ctx.  xc [G][n_ctx][F], yc [G][n_ctx], fp32.
 * Replaces ARTabPFNPredictor.prefill_context / prefill_context_shared and
 * _layer_forward_with_cache(_shared) (ar_tabpfn/model/inference.py:144-223, 579-685). */
ARTAB_API int artab_prefill(const artab_model* m, artab_state* st, const float* xc, const float* yc,
                  int n_feat, void* stream);

/* One autoregressive decode step t for all streams: embeds [buffer(t-1), target(t)]
 * (target only at t = 0), runs every layer (in-place append of the buffer token's
 * K/V, shared-context + private-buffer attention merged by log-sum-exp), applies
 * the final norm and the mixture head and draws y_t.
 *   xt [B][Nt][F]; samples [B][Nt] (column t-1 is read, column t written);
 *   expo [B][K] Exp(1) variates and normal [B] N(0,1) variates of this step;
 *   logdens [B][Nt] (may be NULL) log density of the drawn value; comp [B][Nt] (may be NULL).
 * st->buffer_len is advanced by one when t > 0.
 * Replaces autoregressive_decode / transformer_decode / _layer_decode_with_cache_shared
 * and MixtureGaussianHead.sample (ar_tabpfn/model/inference.py:226-320, 746-833;
 * ar_tabpfn/model/model.py:251-266). */
ARTAB_API int artab_decode_step(const artab_model* m, artab_state* st, const float* xt, int n_feat, int n_targets,
                      int t, float* samples, const float* expo, const float* normal,
                      float* logdens, int32_t* comp, void* stream);

/* Decode step on caller-provided embeddings x_in [B][N][D] (N = 1 or 2; token 0 of
 * an N = 2 step is the buffer token).  Writes z_out [B][N][D] (after the final norm)
 * and commits `commit` (0 or N-1) buffer rows.
 * Replaces ARTabPFNPredictor.transformer_decode (ar_tabpfn/model/inference.py:226-276). */
ARTAB_API int artab_decode_embedded(const artab_model* m, artab_state* st, const float* x_in, int n_new, int commit,
                          float* z_out, void* stream);

/* Teacher-forced joint log density of all targets in one pass:
 * tokens [Buffer_0..Buffer_{Nt-1}, Target_0..Target_{Nt-1}] per stream, block-causal
 * visibility (buffer j sees context + buffers <= j, target i sees context + buffers < i).
 *   xt [B][Nt][F], yt [B][Nt]; logdens [B][Nt].
 * Uses st->kv_buf (needs max_buf >= Nt) as the buffer K/V store; buffer_len is left at Nt.
 * Replaces _evaluate_joint_density_shared/_flex, _teacher_forcing_decode(_shared),
 * _layer_teacher_forcing_shared and MixtureGaussianHead.log_likelihood
 * (ar_tabpfn/model/inference.py:392-488, 835-890; ar_tabpfn/model/model.py:241-272). */
ARTAB_API int artab_teacher_forcing(const artab_model* m, artab_state* st, const float* xt, const float* yt,
                          int n_feat, int n_targets, float* logdens, void* stream);

/* Masked forward over [Buffer_0..Buffer_{Nb-1}, Target_0..Target_{Nt-1}] per stream with a
 * per-token prefix mask on the buffer rows: token j (0 <= j < Nb + Nt) sees the whole context
 * and buffer rows [0, visible[j]) (counts above Nb are clamped).  Buffer row j carries
 * ar_tokens[j], so Nb <= S.  This is the row mask of the reference's training forward
 * restricted to what it can express for the non-context rows: context rows see the context
 * only (artab_prefill), buffer j sees buffers <= j (visible[j] = j + 1), target t sees
 * buffers <= t mod Nb while t < attending_chunks * Nb and none after.
 *   xb [B][Nb][F], yb [B][Nb], xt [B][Nt][F], yt [B][Nt], visible [Nb+Nt] int32 (device);
 *   logdens [B][Nt] log density of yt under the mixture of every target row.
 * Needs max_buf >= Nb; buffer_len is left at Nb.
 * Replaces ARTabPFN.forward / TwoStageTransformer.forward under create_row_mask for
 * inference (ar_tabpfn/model/model.py:317-369, 134-147; ar_tabpfn/model/attention.py:86-175). */
ARTAB_API int artab_forward_masked(const artab_model* m, artab_state* st, const float* xb, const float* yb,
                         const float* xt, const float* yt, int n_feat, int n_buf, int n_targets,
                         const int32_t* visible, float* logdens, void* stream);

/* ------------------------------ single operators -------------------------- */

/* Shared-context attention with LSE output.
 *   q [rows][H][Dh] (dtype), k_ctx [G][H][Ncp][Dh], v_ctx (layout per dtype, see artab_state),
 *   rows_per_group: rows r belong to context group r / rows_per_group (ignored when G = 1);
 *   out [rows][H][Dh] fp32 (normalised), lse [rows][H] fp32 (natural log).
 *   n_splits >= 1 splits the key axis; out/lse then hold n_splits partials
 *   ([split][rows][H][Dh] / [split][rows][H]) to be merged by artab_buffer_attention_merge.
 * Replaces triton_context_attention(_multiq) / pytorch_context_attention
 * (ar_tabpfn/model/triton_kernels.py:347-475, 532-567). */
ARTAB_API int artab_context_attention(int dtype, const void* q, const void* k_ctx, const void* v_ctx,
                            int rows, int rows_per_group, int n_groups, int n_heads, int head_dim,
                            int n_ctx, int n_ctx_pad, int n_splits, float* out, float* lse,
                            int32_t* status, void* stream);

/* Context attention split over n_splits key ranges and merged, with NO caller scratch.
 * (No counterpart in the reference: an addition for callers that cannot allocate.)
 * Same result as artab_context_attention(n_splits) + artab_buffer_attention_merge without
 * buffer keys, but the per-split partials live in a fixed 8 MiB device array inside the
 * library image, so the caller passes inputs and the output only.  For hosts that must not
 * allocate device memory at call time (a pre-sized serving arena, a plugin that is handed
 * tensors but owns no allocator, a latency path where cudaMalloc would stall the device).
 *   out [rows][H][Dh] fp32 (normalised, all splits merged).
 * Limit: n_splits * rows * n_heads * (head_dim + 1) <= 2 097 152 floats, else ARTAB_ECAPACITY.
 * The first call on each device looks the array's device address up (a host-side, one-off
 * set-up step): make that first call outside any stream capture.  All calls on a device share
 * the one array: calls whose kernels may overlap on the GPU (different streams) race on it;
 * serialise them.  Every GPU that loads the library holds the 8 MiB until the process exits.
 * The status word of the bounded waits also lives in the array, out of the caller's reach: if a
 * wait of the contraction gives up, every element of `out` is NaN (never a mix of stale partials),
 * which is how such a call reports the failure. */
ARTAB_API int artab_context_attention_noalloc(int dtype, const void* q, const void* k_ctx, const void* v_ctx,
                                              int rows, int rows_per_group, int n_groups, int n_heads,
                                              int head_dim, int n_ctx, int n_ctx_pad, int n_splits, float* out,
                                              void* stream);

/* Private-buffer attention pass + log-sum-exp merge with the context partials.
 * One work item per (stream, head, item): up to two queries (a "target" row and a
 * "buffer" row, -1 = absent) attend to keys [0, len) of that stream-head's span in
 * kv_buf and are merged in registers with n_splits context partials.
 *   decode  (items_per_stream = 1): target row = b*n_new + n_new-1, buffer row = b*n_new (n_new = 2), len = len0
 *   teacher forcing (items_per_stream = Nt+1): item i: target row b*2Nt+Nt+i (i < Nt),
 *            buffer row b*2Nt+i-1 (i >= 1), len = i
 *   out [rows][H][Dh] fp32.
 * Replaces pytorch_buffer_attention, pytorch_teacher_forcing_buffer_attention,
 * merge_attention_outputs and the torch.cat of K/V in the decode layer
 * (ar_tabpfn/model/triton_kernels.py:478-524, 570-659; ar_tabpfn/model/inference.py:802-814). */
ARTAB_API int artab_buffer_attention_merge(int dtype, const void* q, const void* kv_buf, int n_streams, int n_heads,
                                 int head_dim, int max_buf, int mode_tf, int n_new_or_nt, int len0,
                                 const float* o_part, const float* lse_part, int n_splits, int rows,
                                 float* out, void* stream);

/* The general prefix form: every stream carries `tokens_per_stream` query rows, and row j of a
 * stream sees the first visible[j] of the stream's n_buf buffer rows (int32 device array
 * [tokens_per_stream], values clamped to [0, n_buf]); merged in registers with the n_splits context
 * partials like the other forms.  This is the buffer half of the reference's row attention under
 * create_row_mask (ar_tabpfn/model/attention.py:86-175), where the visibility of the buffer rows is
 * a prefix for every non-context row; the context half is artab_context_attention.
 * key_mask (optional, may be NULL): [rows][H][max_buf] bytes, non-zero = this query sees that buffer
 * key, applied on top of the prefix: with visible[j] = n_buf it expresses ANY boolean mask, which is
 * what pytorch_buffer_attention / hybrid_attention accept (ar_tabpfn/model/triton_kernels.py:570-614).
 *   out [rows][H][Dh] fp32, rows = n_streams * tokens_per_stream; lse_out optional [rows][H] fp32
 *   (natural log of the merged attention, -inf where a query sees nothing). */
ARTAB_API int artab_buffer_attention_merge_visible(int dtype, const void* q, const void* kv_buf, int n_streams,
                                                   int n_heads, int head_dim, int max_buf, int tokens_per_stream,
                                                   const int32_t* visible, int n_buf, const uint8_t* key_mask,
                                                   const float* o_part, const float* lse_part, int n_splits,
                                                   int rows, float* out, float* lse_out, void* stream);

/* The decode form of artab_buffer_attention_merge with RAGGED private buffers: stream b sees
 * its first lens[b] buffer rows (int32 device array [B], values clamped to [0, len_max];
 * NULL: len_max for every stream), the same for every head and for both queries of a stream.
 * This is pytorch_buffer_attention's / hybrid_attention's `mask` argument when the mask is a
 * per-stream length (the reference's own masked test case and the ragged 0..63-key buffers
 * of its decode-attention micro-benchmark).  A query with no visible buffer row and no
 * finite context partial gives out = 0.
 *   lse_out [rows][H] fp32 (may be NULL): natural-log LSE of the merged attention, -inf when
 *   nothing is visible; with one context partial of lse = -inf this is the buffer attention's
 *   own LSE, which makes the call pytorch_buffer_attention.
 * Replaces pytorch_buffer_attention with a mask, merge_attention_outputs
 * (ar_tabpfn/model/triton_kernels.py:570-614, 478-524) and hybrid_attention's buf_mask
 * (ar_tabpfn/model/triton_kernels.py:705-755). */
ARTAB_API int artab_buffer_attention_merge_ragged(int dtype, const void* q, const void* kv_buf, int n_streams,
                                        int n_heads, int head_dim, int max_buf, int n_new, const int32_t* lens,
                                        int len_max, const float* o_part, const float* lse_part, int n_splits,
                                        int rows, float* out, float* lse_out, void* stream);

/* In-place append of one new K/V row per (stream, head) at position `pos`.
 *   k_new, v_new [B][H][Dh] (dtype).
 * Replaces the slice assignment into k_buf_cache / v_buf_cache
 * (ar_tabpfn/model/inference.py:816-821). */
ARTAB_API int artab_kv_append(int dtype, void* kv_buf, const void* k_new, const void* v_new, int n_streams, int n_heads,
                    int head_dim, int max_buf, int pos, void* stream);

/* Embedder: out[r][:] = mean_F(x[r][:]) * wx + bx (+ y[r] * wy + by) + marker[kind] (+ ar_tokens[ar_idx[r]]).
 *   x [rows][F], y [rows] or NULL, ar_idx [rows] or NULL.
 * Replaces Embedder.embed_context / embed_buffer / embed_target (ar_tabpfn/model/model.py:51-76). */
ARTAB_API int artab_embed(const artab_model* m, const float* x, const float* y, const int32_t* ar_idx, int rows,
                int n_feat, int kind, float* out, void* stream);

/* Mixture head on z [rows][D] (already normalised): log density of y [rows] -> logdens [rows].
 * Replaces MixtureGaussianHead.log_likelihood (ar_tabpfn/model/model.py:190-209, 241-272). */
ARTAB_API int artab_head_logpdf(const artab_model* m, const float* z, const float* y, int rows, float* logdens,
                      void* stream);

/* Mixture head on z [rows][D]: draw y with variates expo [rows][K], normal [rows].
 * Replaces MixtureGaussianHead.sample (ar_tabpfn/model/model.py:251-266). */
ARTAB_API int artab_head_sample(const artab_model* m, const float* z, const float* expo, const float* normal, int rows,
                      float* y, float* logdens, int32_t* comp, void* stream);

/* ------------------------------ utilities -------------------------------- */

/* Number of key splits artab_decode_step / artab_teacher_forcing will use for `rows`
 * query rows (workspace sizing). */
ARTAB_API int artab_plan_splits(int dtype, int rows, int rows_per_group, int n_groups, int n_heads, int n_ctx);

/* Per-launch timing for benchmarks: after artab_profile_enable(1) every kernel launch of
 * this library (on the calling thread) is bracketed by CUDA events on its stream.
 * artab_profile_read (call after synchronising) sums elapsed milliseconds and launch
 * counts per kernel kind (0 embed, 1 per-token dense chain, 2 context attention,
 * 3 buffer pass + merge, 4 KV append), clears the record and returns the number read. */
ARTAB_API void artab_profile_enable(int on);
ARTAB_API int artab_profile_read(double* ms_per_kind, int64_t* launches_per_kind, int n_kinds);

/* Programmatic dependent launch (on by default, process-wide): the kernels of the decode
 * chain are launched so that each may begin its set-up and weight prefetch while the kernel
 * before it in the stream drains, and the private-buffer pass runs beside the context
 * contraction; results are bit-identical either way.  Pass 0 to launch every kernel fully
 * serialised (diagnostics); the environment variable ARTAB_DEPENDENT_LAUNCH=0 sets that
 * default at load time, for profilers that replay single kernels.  No counterpart in the
 * reference. */
ARTAB_API void artab_set_dependent_launch(int on);

/* Diagnostics of the bounded device-side waits (process-wide, off by default; no counterpart in
 * the reference).  Every mbarrier wait inside the tensor-core kernels gives up after a limit, the
 * CTA then writes nothing more, frees what it holds, sets the status word and returns.
 *   ARTAB_DEBUG_WAIT_CYCLES        value = limit in SM clock cycles for the context contraction's waits
 *                                  (0 restores the built-in limit of about one second)
 *   ARTAB_DEBUG_DROP_SCORE_COMMITS value != 0: the context contraction's MMA thread never signals
 *                                  "scores ready", so its softmax threads' waits run out.  This is how
 *                                  the tests exercise the give-up path without faulting anything:
 *                                  the kernel returns normally, status is non-zero, `out` untouched. */
#define ARTAB_DEBUG_WAIT_CYCLES 0
#define ARTAB_DEBUG_DROP_SCORE_COMMITS 1
ARTAB_API int artab_debug_set(int key, long long value);

/* Kernels launched by this library on the calling thread since the last reset
 * (a host-side counter for benchmarks). */
ARTAB_API int64_t artab_launch_count(void);
ARTAB_API void artab_launch_count_reset(void);

/* Text of the last error on the calling thread (never NULL). */
ARTAB_API const char* artab_last_error(void);

/* Library build tag, e.g. "artab-b200 sm_100a". */
ARTAB_API const char* artab_version(void);

#ifdef __cplusplus
}
#endif
#endif /* ARTAB_H_ */
