// Where a freshly projected K or V element of token row `row`, model column `c` goes:
// the context cache during prefill, the private buffer cache (in-place append) otherwise.
#pragma once
#include "common.cuh"

namespace artab {

template <typename T>
__device__ __forceinline__ void scatter_k(const KvDest& kv, long row, int c, float val) {
  const int h = c / kv.head_dim, d = c - h * kv.head_dim;
  if (kv.mode == KV_PREFILL) {
    const long g = row / kv.n_ctx, i = row - g * kv.n_ctx;
    reinterpret_cast<T*>(kv.k_ctx)[((size_t)(g * kv.n_heads + h) * kv.n_ctx_pad + i) * kv.head_dim + d] =
        from_f32<T>(val);
  } else {
    const long b = row / kv.tokens_per_stream;
    const int j = (int)(row - b * kv.tokens_per_stream);
    if (j >= kv.n_kv_tokens) return;
    reinterpret_cast<T*>(kv.kv_buf)[(((size_t)(b * kv.n_heads + h) * kv.max_buf + kv.pos0 + j) * 2) * kv.head_dim + d] =
        from_f32<T>(val);
  }
}

template <typename T>
__device__ __forceinline__ void scatter_v(const KvDest& kv, long row, int c, float val) {
  const int h = c / kv.head_dim, d = c - h * kv.head_dim;
  if (kv.mode == KV_PREFILL) {
    const long g = row / kv.n_ctx, i = row - g * kv.n_ctx;
    if (kv.dtype == ARTAB_BF16) {  // transposed, split into a bf16 hi and lo part: [.., 2*Dh][Ncp]
      T* vb = reinterpret_cast<T*>(kv.v_ctx) + ((size_t)(g * kv.n_heads + h) * 2 * kv.head_dim) * kv.n_ctx_pad + i;
      const T hi = from_f32<T>(val);
      vb[(size_t)d * kv.n_ctx_pad] = hi;
      vb[(size_t)(kv.head_dim + d) * kv.n_ctx_pad] = from_f32<T>(val - to_f32<T>(hi));
    } else {
      reinterpret_cast<T*>(kv.v_ctx)[((size_t)(g * kv.n_heads + h) * kv.n_ctx_pad + i) * kv.head_dim + d] =
          from_f32<T>(val);
    }
  } else {
    const long b = row / kv.tokens_per_stream;
    const int j = (int)(row - b * kv.tokens_per_stream);
    if (j >= kv.n_kv_tokens) return;
    reinterpret_cast<T*>(
        kv.kv_buf)[(((size_t)(b * kv.n_heads + h) * kv.max_buf + kv.pos0 + j) * 2 + 1) * kv.head_dim + d] =
        from_f32<T>(val);
  }
}

}  // namespace artab
