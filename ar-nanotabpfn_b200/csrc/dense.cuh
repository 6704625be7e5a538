// Host-visible argument blocks of the row-local ("per token") kernels.
#pragma once
#include "common.cuh"

namespace artab {

// Which rows the embedder produces and where their inputs come from.
enum EmbedMode : int { EMB_ROWS = 0, EMB_DECODE = 1, EMB_TF = 2, EMB_FWD = 3 };

struct EmbedArgs {
  int mode, rows, D, F, kind;
  const float *wx, *bx, *wy, *by, *marker, *ar_tokens;
  // EMB_ROWS
  const float* x;        // [rows][F]
  const float* y;        // [rows] or null
  const int32_t* ar_idx; // [rows] or null
  // EMB_DECODE / EMB_TF
  const float* xt;       // [B][Nt][F]
  const float* yt;       // decode: samples [B][Nt]; tf: yt [B][Nt]
  int Nt, t, n_new, S;
  // EMB_FWD: per stream [Buffer_0..Buffer_{Nb-1}, Target_0..Target_{Nt-1}], buffer rows from their own arrays
  const float* xb;       // [B][Nb][F]
  const float* yb;       // [B][Nb]
  int Nb;
  float* out;            // [rows][D]
  int out_lane_major;    // write `out` in the lane-major layout the tensor-core chain reads (padded workspace)
};

struct DenseArgs {
  int rows, D, Dff, n_comp;
  int do_post, do_final, do_head, do_pre;
  artab_layer_weights post_w, pre_w;
  int lane_major;      // tensor-core chain: attn and the x1 workspace use the lane-major layout
  int x_in_lane_major; // tensor-core chain: x_in was written in that layout too (by the embedder)
  const float* attn;   // [rows][D]  post input
  const float* x1_in;  // [rows][D]  post residual input
  const float* x_in;   // [rows][D]  chain input when !do_post
  float* x_out;        // [rows][D]  layer output (optional)
  float* x1_out;       // [rows][D]  pre output
  void* q_out;         // [rows][D]  pre output, cache dtype
  KvDest kv;
  const float *lnf_g, *lnf_b, *wa_t, *ba, *wb_t, *bb, *mean_bias, *std_bias, *weight_bias;
  float* z_out;        // [rows][D] optional
  int head_mode;       // 0 none, 1 sample, 2 log-pdf
  int head_tps, head_first, out_stride, out_col;
  const float *expo, *normal, *y_in;
  float* y_out;
  float* ld_out;
  int32_t* comp_out;
  int32_t* status;     // device status word (bounded waits), may be null
  // tensor-core chain: scratch for the CTA-pair exchange, pair_slots slots of pair_slot_stride floats
  // (>= rows rounded up to 128, times D, each); null: one CTA per row tile
  float* pair_scratch;
  size_t pair_slot_stride;
  int pair_slots;      // slots in pair_scratch; a pair uses 6: MLP exchange (0, 1), head exchange (2, 3), parking (4, 5)
  const void *tc_wa, *tc_wb;  // tensor-core tiles of the head matrices (null: fp32 chain)
  int tc_head_lo;
#ifdef ARTAB_TIMELINE
  int tl_slot;         // diagnostic builds: which timeline slot this launch stamps
#endif
};

int launch_embed(const EmbedArgs& a, cudaStream_t s);
int launch_dense(const DenseArgs& a, cudaStream_t s);     // picks the tensor-core chain when it applies
int launch_dense_tc(const DenseArgs& a, cudaStream_t s);  // tcgen05 chain (bf16 mode)
bool dense_tc_applicable(const DenseArgs& a);

}  // namespace artab
