// Split-context attention without caller-provided scratch.
//
// artab_context_attention_noalloc runs the same two kernels as
// artab_context_attention (n_splits > 1) followed by artab_buffer_attention_merge
// (no buffer keys), but keeps the per-split partial outputs in a fixed device
// array that is part of this library image instead of in memory the caller
// allocates.  It is meant for hosts that may not allocate device memory at the
// point of the call: code running inside a pre-sized serving arena, inside a
// stream-ordered region where a cudaMalloc would synchronise the device, or a
// plugin that is handed input and output tensors only and owns no allocator.
#include <cstring>

#include "attn.cuh"

namespace artab {
namespace {

// 8 MiB of partials: n_splits * rows * n_heads * (head_dim + 1) floats must fit.
constexpr size_t kScratchFloats = 2u << 20;
static __device__ __align__(256) float g_noalloc_scratch[kScratchFloats + 64];  // + status word

float* g_scratch_ptr[kMaxDevices] = {nullptr};

// The array's name is only a host-side handle; kernels need its device address.
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  ARTAB_REQUIRE(e == cudaSuccess && dev >= 0 && dev < kMaxDevices, ARTAB_ELAUNCH, "noalloc: cudaGetDevice failed: %s",
                cudaGetErrorString(e));
  if (!g_scratch_ptr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    ARTAB_REQUIRE(e == cudaSuccess && p, ARTAB_ELAUNCH, "noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                  cudaGetErrorString(e));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return ARTAB_OK;
}

}  // namespace
}  // namespace artab

using namespace artab;

extern "C" ARTAB_API int artab_context_attention_noalloc(int dtype, const void* q, const void* k_ctx,
                                                         const void* v_ctx, int rows, int rows_per_group,
                                                         int n_groups, int n_heads, int head_dim, int n_ctx,
                                                         int n_ctx_pad, int n_splits, float* out, void* stream) {
  PlainLaunchScope plain;  // the caller's earlier launches are unknown: see common.cuh
  ARTAB_REQUIRE(q && k_ctx && v_ctx && out, ARTAB_EINVAL, "context_attention_noalloc: null pointer");
  ARTAB_REQUIRE(rows >= 1 && n_groups >= 1 && n_heads >= 1 && n_ctx >= 1 && n_splits >= 1 && n_ctx_pad >= n_ctx,
                ARTAB_EINVAL, "context_attention_noalloc: bad sizes");
  ARTAB_REQUIRE(n_groups == 1 || rows == rows_per_group * n_groups, ARTAB_EINVAL,
                "context_attention_noalloc: rows must equal rows_per_group * n_groups");
  const size_t need = (size_t)n_splits * rows * n_heads * (head_dim + 1);
  ARTAB_REQUIRE(need <= kScratchFloats, ARTAB_ECAPACITY,
                "context_attention_noalloc: n_splits * rows * n_heads * (head_dim + 1) = %zu floats exceeds the "
                "built-in scratch of %zu floats (8 MiB); use artab_context_attention with caller memory",
                need, kScratchFloats);
  float* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  float* o_part = scratch;
  float* lse_part = scratch + (size_t)n_splits * rows * n_heads * head_dim;
  int32_t* status = reinterpret_cast<int32_t*>(scratch + kScratchFloats);
  // the array keeps the previous call's contents: partials are fully rewritten below,
  // only the status word has to start at zero
  cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int32_t), s);
  ARTAB_REQUIRE(e == cudaSuccess, ARTAB_ELAUNCH, "noalloc: status clear failed: %s", cudaGetErrorString(e));

  CtxAttnArgs c;
  memset(&c, 0, sizeof(c));
  c.dtype = dtype;
  c.q = q;
  c.k_ctx = k_ctx;
  c.v_ctx = v_ctx;
  c.v_transposed = dtype == ARTAB_BF16;
  c.rows = rows;
  c.rows_per_group = rows_per_group;
  c.n_groups = n_groups;
  c.n_heads = n_heads;
  c.head_dim = head_dim;
  c.n_ctx = n_ctx;
  c.n_ctx_pad = n_ctx_pad;
  c.n_splits = n_splits;
  c.scale = 1.0f / sqrtf((float)head_dim);
  c.out = o_part;
  c.lse = lse_part;
  c.status = status;
  rc = ctx_attn_tc_supported(dtype, head_dim) ? launch_ctx_attn_tc(c, s) : launch_ctx_attn_simt(c, s);
  if (rc) return rc;

  BufMergeArgs b;
  memset(&b, 0, sizeof(b));
  b.dtype = dtype;
  b.q = q;
  b.kv_buf = nullptr;
  b.n_heads = n_heads;
  b.head_dim = head_dim;
  b.max_buf = 0;
  b.mode_tf = 0;
  b.n_new = 1;
  b.len0 = 0;
  b.n_items = (long)rows * n_heads;
  b.o_part = o_part;
  b.lse_part = lse_part;
  b.n_splits = n_splits;
  b.rows = rows;
  b.scale = c.scale;
  b.out = out;
  b.poison_if = status;  // a wait that gave up in the contraction turns the whole output into NaN
  return launch_buf_merge(b, s);
}
