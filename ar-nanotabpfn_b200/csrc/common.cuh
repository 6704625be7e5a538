// Shared helpers for the artab sm_100a kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "artab.h"

namespace artab {

// ---- error plumbing (host) ------------------------------------------------
void set_error(const char* fmt, ...);
int check_launch(const char* what);
void count_launch();
// per-launch CUDA-event timing, active only after artab_profile_enable(1)
enum ProfKind : int { PROF_EMBED = 0, PROF_DENSE = 1, PROF_CTX = 2, PROF_BUF = 3, PROF_APPEND = 4, PROF_KINDS = 5 };
void prof_begin(int kind, cudaStream_t s);
void prof_end(cudaStream_t s);

// ---- programmatic dependent launch ---------------------------------------------
// Kernels of the decode chain are launched with the programmatic-stream-serialization attribute:
// a kernel may start while its predecessor in the stream still runs, does the work that needs
// nothing from it (barrier set-up, tensor-memory allocation, loads of weights), and then executes
// dep_wait(), which returns once the predecessor grid has completed and its writes are visible.
// Rules every such kernel follows: (1) it calls dep_wait() before it reads anything an earlier
// kernel wrote and before it writes global memory; (2) it calls dep_trigger() only after its own
// dep_wait(), so a dependent that starts early knows that everything older than its predecessor
// has completed.  One exception to (2): the buffer-pass kernels trigger at their start, because
// their dependent is always a dense chain, which touches only model constants before its own wait
// (and that wait still covers everything older: a buffer-pass grid completes only after its own
// wait).  Without the launch attribute both calls are no-ops.
//
// What each kernel reads BEFORE its dep_wait() (the work it overlaps with its predecessor):
//   embed_kernel            nothing
//   dense_tc_kernel         weight tiles, LayerNorm vectors and biases (model constants)
//   ctx_attn_tc_kernel      context K / V tiles, only when the caller says they are stable (kv_stable)
//   buf_mma_kernel /
//   buf_merge_kernel        q, the private K / V rows and the per-stream lengths
// The last line is safe only where the launch BEFORE the predecessor produced q and the K / V rows,
// which holds inside artab_prefill / artab_decode_step / artab_teacher_forcing / artab_forward_masked
// (embed, dense chain, context contraction, buffer pass: the buffer pass's predecessor is the context
// contraction, which waits before it triggers).  The single-operator entry points cannot know what
// the caller launched before them, so they launch every kernel plainly (PlainLaunchScope): the
// kernel then starts after everything earlier in the stream has completed and the rule is moot.
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dep_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#ifdef ARTAB_TIMELINE
// Diagnostic builds only: a log of global-timer stamps shared by every kernel of the library, read
// with artab_debug_stamps.  Every CTA of a grid of up to
// ARTAB_STAMP_ALL CTAs, else the first and the last CTA, records (kernel, event, CTA, ns).
// Kernels: 0 embed, 1 tensor-core dense chain, 2 context contraction, 3 buffer pass (tensor-core
// fragments), 4 buffer pass (scalar); events: 0 entry, 1 predecessor complete, 2 end, 3 kernel-specific
// (buffer pass: private keys done, before the wait; dense chain: last instruction).
#ifndef ARTAB_STAMP_ALL
#define ARTAB_STAMP_ALL 32   // grids up to this many CTAs record every CTA
#endif
struct StampLog {
  unsigned long long n;
  long long rec[1 << 16][2];
};
StampLog* stamp_log_buffer();       // one device buffer per process, allocated on first use
static __device__ StampLog* g_stamp_log;   // one copy per translation unit, attached before its launches
static inline void stamp_log_attach() {
  static bool done = false;
  if (done) return;
  StampLog* p = stamp_log_buffer();
  cudaMemcpyToSymbol(g_stamp_log, &p, sizeof p);
  done = true;
}
__device__ __forceinline__ void stamp(int kernel, int event) {
  const unsigned nb = gridDim.x * gridDim.y * gridDim.z;
  const unsigned b = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  StampLog* log = g_stamp_log;
  if (!log || (nb > ARTAB_STAMP_ALL && b != 0 && b != nb - 1)) return;
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  const unsigned long long i = atomicAdd(&log->n, 1ULL);
  if (i < (1ULL << 16)) {
    log->rec[i][0] = kernel * 10000 + event * 1000 + (nb > ARTAB_STAMP_ALL ? (b ? 999 : 0) : (int)b);
    log->rec[i][1] = t;
  }
}
#define ARTAB_STAMP(kernel, event) stamp(kernel, event)
#define ARTAB_STAMP_ATTACH() stamp_log_attach()
#else
#define ARTAB_STAMP(kernel, event) do { } while (0)
#define ARTAB_STAMP_ATTACH() do { } while (0)
#endif

bool dependent_launch_enabled();
// diagnostics set through artab_debug_set: limit of the bounded waits (0: the built-in second or so) and
// the switch that makes the context kernel's waits run out (see artab.h)
long long debug_wait_cycles();
int debug_drop_score_commits();

// While one of these lives on the calling thread, launch_dependent* issue plain launches.
struct PlainLaunchScope {
  PlainLaunchScope();
  ~PlainLaunchScope();
  PlainLaunchScope(const PlainLaunchScope&) = delete;
  PlainLaunchScope& operator=(const PlainLaunchScope&) = delete;
};

// Largest dynamic shared-memory size a kernel has been configured for, per device: the opt-in is a
// per-device attribute, so a process that uses several GPUs repeats it on each.
constexpr int kMaxDevices = 64;
struct SmemConfig {
  size_t bytes[kMaxDevices] = {};
  // several_per_sm: the kernel is meant to have more than one CTA resident per SM, so it also asks
  // for the largest shared-memory carve-out (the default heuristic may pick one that fits a single CTA)
  template <typename K>
  cudaError_t ensure(K kernel, size_t smem, bool several_per_sm = false) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const bool tracked = dev >= 0 && dev < kMaxDevices;
    if (tracked && smem <= bytes[dev]) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess && several_per_sm)
      e = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess && tracked) bytes[dev] = smem;
    return e;
  }
};

// cluster_x > 1 launches thread-block clusters of that many CTAs along x (grid.x a multiple of it).
template <typename... P, typename... A>
inline cudaError_t launch_dependent_cluster(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                            unsigned cluster_x, A&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (dependent_launch_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<P>(args)...);
}

template <typename... P, typename... A>
inline cudaError_t launch_dependent(void (*kernel)(P...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                    A&&... args) {
  return launch_dependent_cluster(kernel, grid, block, smem, s, 1u, static_cast<A&&>(args)...);
}

#define ARTAB_REQUIRE(cond, code, ...) \
  do {                                 \
    if (!(cond)) {                     \
      ::artab::set_error(__VA_ARGS__); \
      return (code);                   \
    }                                  \
  } while (0)

// ---- storage-type conversion ------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// 16-byte vector of storage elements -> floats
template <typename T>
struct Vec16;
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void unpack(const uint4& v, float* out) {
    out[0] = __uint_as_float(v.x); out[1] = __uint_as_float(v.y);
    out[2] = __uint_as_float(v.z); out[3] = __uint_as_float(v.w);
  }
  __device__ static __forceinline__ void load(const float* p, float* out) {
    unpack(*reinterpret_cast<const uint4*>(p), out);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void load(const __nv_bfloat16* p, float* out) {
    unpack(*reinterpret_cast<const uint4*>(p), out);
  }
  __device__ static __forceinline__ void unpack(const uint4& v, float* out) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// "Lane-major" layout of a [rows][D] fp32 workspace: 32-row tiles, inside a tile the float4 column
// groups are outermost and the 32 rows innermost, so that 32 threads owning 32 consecutive rows
// (tensor-memory lanes) read or write one contiguous 512-byte span per float4.
__host__ __device__ __forceinline__ size_t lane_major_index(long row, int col, int D) {
  return ((size_t)(row >> 5) * (D >> 2) + (col >> 2)) * 128 + (size_t)(row & 31) * 4 + (col & 3);
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---- how a dense kernel scatters freshly projected K / V rows -----------------
enum KvMode : int { KV_NONE = 0, KV_PREFILL = 1, KV_DECODE = 2, KV_TF = 3 };

struct KvDest {
  int mode;          // KvMode
  int dtype;         // ARTAB_F32 / ARTAB_BF16
  int n_heads, head_dim;
  // prefill: rows = G * n_ctx, row r -> (g = r / n_ctx, i = r % n_ctx)
  void* k_ctx;       // [G][H][Ncp][Dh]   (this layer)
  void* v_ctx;       // fp32 [G][H][Ncp][Dh] / bf16 [G][H][Dh][Ncp]
  int n_ctx, n_ctx_pad;
  // decode / teacher forcing: rows = B * tokens_per_stream
  void* kv_buf;      // [B][H][T][2][Dh]  (this layer)
  int max_buf;
  int tokens_per_stream;  // decode: n_new (1 or 2); tf: 2*Nt
  int n_kv_tokens;        // decode: n_new-1 (0 or 1) leading tokens are buffer rows; tf: Nt
  int pos0;               // decode: buffer_len (position of the appended row); tf: 0
};

}  // namespace artab
