// Argument blocks of the attention kernels.
#pragma once
#include "common.cuh"

namespace artab {

struct CtxAttnArgs {
  int dtype;
  const void* q;      // [rows][H][Dh]
  const void* k_ctx;  // [G][H][Ncp][Dh]
  const void* v_ctx;  // [G][H][Ncp][Dh] or transposed [G][H][Dh][Ncp]
  int v_transposed;
  int rows, rows_per_group, n_groups, n_heads, head_dim, n_ctx, n_ctx_pad, n_splits;
  float scale;
  float* out;         // [splits][rows][H][Dh]
  int out_lane_major; // n_splits == 1 only: write the [rows][H*Dh] result in the lane-major layout
  float* lse;         // [splits][rows][H]
  int32_t* status;    // device status word (bounded waits), may be null for SIMT
  int kv_stable;      // k_ctx / v_ctx were not written by the kernel launched just before this one
};

struct BufMergeArgs {
  int dtype;
  const void* q;       // [rows][H][Dh]
  const void* kv_buf;  // [B][H][T][2][Dh]
  int n_heads, head_dim, max_buf;
  int mode_tf, nt, n_new, len0;  // mode_tf: 0 decode step, 1 teacher forcing, 2 per-token visible prefix
  const int32_t* visible;  // mode 2: [tps] token j of a stream sees buffer keys [0, visible[j])
  int tps;                 // mode 2: tokens per stream
  const uint8_t* key_mask; // mode 2, optional: [rows][H][max_buf] bytes, non-zero = the query sees that buffer key
                           // (on top of the visible prefix): arbitrary boolean masks of the functional API
  const int32_t* lens;     // mode 0: [B] visible buffer rows of each stream, clamped to len0 (null: len0 for all)
  float* lse_out;          // optional [rows][H]: natural-log LSE of the merged attention (-inf: nothing visible)
  long n_items;
  const float* o_part;    // [splits][rows][H][Dh]
  const float* lse_part;  // [splits][rows][H]
  int n_splits, rows;
  float scale;
  float* out;  // [rows][H][Dh]
  int out_lane_major;  // write out in the lane-major layout instead
  // Optional device word: when it is non-zero after the preceding kernel (a bounded wait of the
  // context contraction gave up, so some partials were never written) the merged output is NaN
  // instead of a plausible-looking mix of stale partials.
  const int32_t* poison_if;
};

int launch_ctx_attn_simt(const CtxAttnArgs& a, cudaStream_t s);
int launch_ctx_attn_tc(const CtxAttnArgs& a, cudaStream_t s);  // tcgen05, bf16, head_dim 32
bool ctx_attn_tc_supported(int dtype, int head_dim);
int launch_buf_merge(const BufMergeArgs& a, cudaStream_t s);      // picks the MMA kernel when it applies
int launch_buf_merge_mma(const BufMergeArgs& a, cudaStream_t s);  // mma.sync, bf16, head_dim 32
bool buf_mma_supported(int dtype, int head_dim);
int launch_kv_append(int dtype, void* kv, const void* k_new, const void* v_new, long n_bh, int dh, int max_buf,
                     int pos, cudaStream_t s);

}  // namespace artab
