// Row-local fp32 kernels: embedder, the fused per-token layer chain
// (out-proj + LN2 + MLP + LN3 [+ final LN + mixture head] [+ next layer's
// feature-attention fold + LN1 + QKV + KV-cache scatter]) and the mixture head.
//
// Every token row is independent, so one CTA owns R rows and walks the whole
// chain with the activations resident in shared memory; weights are streamed
// from L2 with coalesced reads (they are stored [in][out]).  All arithmetic is
// plain fp32 FMA: this is the path that has to agree with the fp32 CPU
// reference to 1e-5 on the log density, so no TF32 / bf16 operand rounding.
#include "dense.cuh"
#include "kv_scatter.cuh"

namespace artab {

namespace {

constexpr int kRows = 8;  // rows per CTA

// Dynamic shared memory of the chain kernel.  Everything is addressed as an offset into this
// array so that the compiler emits shared-space loads with 32-bit address arithmetic.
extern __shared__ __align__(128) float g_smem[];

__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)); }

// ---------------------------------------------------------------------------
// Weight streaming.  The chain's GEMMs run back to back over the same R rows, so
// the CTA walks one fixed schedule of weight slabs (KC consecutive rows of a
// [K][N] matrix = one contiguous span).  A dedicated producer warp keeps kNBuf
// bulk copies (cp.async.bulk, completion on an mbarrier) in flight into a
// shared-memory ring, across GEMM and LayerNorm boundaries; the compute warps
// consume slab by slab and hand ring slots back through "empty" mbarriers, so
// no CTA-wide barrier sits between slabs.
// ---------------------------------------------------------------------------
constexpr int kNBuf = 6;
constexpr int kBufBytes = 24576;
constexpr long long kWaitCycles = 2000000000LL;

struct Stream {
  uint64_t full[kNBuf];
  uint64_t empty[kNBuf];
  int abort_flag;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool mbar_try(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(b)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait; false once the CTA is aborting (its results are void and the status word is set).
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(b, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try(b, parity)) {
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      return false;
    }
  }
  return true;
}

// compute threads only (the producer warp never joins)
__device__ __forceinline__ void sync_compute(int n_threads) { asm volatile("bar.sync 1, %0;" ::"r"(n_threads) : "memory"); }

// columns-per-thread / k-split plan for an [R x K] . [K x N] product on T threads.  `cap` = columns the
// k-split scratch holds per row ([3][R][D] floats: (ksplit - 1) * N must fit in 3 * D).
// A k-group walks its share of a slab four rows at a time (16-byte reads of the activations), so
// K must be a multiple of 4 * ksplit.
__host__ __device__ inline void plan_gemm(int K, int N, int T, int cap, int& cpt, int& ksplit) {
  for (cpt = 4; cpt >= 1; --cpt) {  // every thread busy: the column groups divide the threads
    if (N % cpt) continue;
    const int cols = N / cpt;
    if (cols <= T && T % cols == 0 && T / cols <= 4 && (T / cols - 1) * N <= cap && K % (4 * (T / cols)) == 0) {
      ksplit = T / cols;
      return;
    }
  }
  ksplit = 1;
  for (cpt = 1; cpt <= 4; ++cpt)    // otherwise the fewest columns per thread that cover N; the rest idle
    if (N % cpt == 0 && N / cpt <= T) return;
  cpt = 1;  // N > 4 T or no divisor: refused on the host (gemm_plan_ok)
}
__host__ __device__ inline bool gemm_plan_ok(int K, int N, int T, int cap) {
  int cpt, ks;
  plan_gemm(K, N, T, cap, cpt, ks);
  return N % cpt == 0 && N / cpt <= T && K % (4 * ks) == 0 && (size_t)4 * ks * N * sizeof(float) <= (size_t)kBufBytes;
}

// rows of W per slab: as many as fit a ring slot, a multiple of 4 per k-group
__host__ __device__ inline int slab_rows(int K, int N, int T, int cap) {
  int cpt, ks;
  plan_gemm(K, N, T, cap, cpt, ks);
  const int q = 4 * ks;
  int kc = (kBufBytes / (4 * N)) / q * q;
  if (kc < q) kc = q;
  return kc > K ? K : kc;
}

// producer: stream every slab of one matrix (lane 0 of the producer warp)
__device__ __forceinline__ bool produce(Stream* st, float* ring, int& issued, const float* w, int K, int N, int T,
                                        int cap) {
  const int kc = slab_rows(K, N, T, cap);
  for (int k0 = 0; k0 < K; k0 += kc) {
    const int rows = min(kc, K - k0);
    const uint32_t bytes = (uint32_t)rows * N * 4u;
    const int buf = issued % kNBuf;
    if (issued >= kNBuf && !mbar_wait(&st->empty[buf], ((issued / kNBuf) + 1) & 1, &st->abort_flag)) return false;
    uint64_t* bar = &st->full[buf];
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(ring + (size_t)buf * (kBufBytes / 4))), "l"(w + (size_t)k0 * N), "r"(bytes),
                 "r"(smem_u32(bar))
                 : "memory");
    ++issued;
  }
  return true;
}

struct Chain {
  Stream* st;
  int scratch;     // offset of the k-split partial sums [ksplit-1][R][N]
  int consumed;    // slabs consumed so far
  int T;           // compute threads
  int cap;         // scratch columns per row (see plan_gemm)
};

// out[r][n] = act(bias[n] + sum_k a[r][k] * W[k][n]) for the CTA's R rows; a and out in shared memory.
template <int R, int CPT>
__device__ __noinline__ void gemm_body(Chain& ch, int K, int N, int ksplit, int a_off, int lda,
                                       const float* __restrict__ bias, bool gelu, int o_off, int ldo) {
  const int cols = (N + CPT - 1) / CPT;
  const int cg = threadIdx.x % cols, kg = threadIdx.x / cols;
  const bool active = kg < ksplit && (CPT > 1 || cg < N);
  const int kc = slab_rows(K, N, ch.T, ch.cap);
  int consumed = ch.consumed;
  float acc[CPT][R];
#pragma unroll
  for (int c = 0; c < CPT; ++c)
#pragma unroll
    for (int r = 0; r < R; ++r) acc[c][r] = 0.f;

  for (int k0 = 0; k0 < K; k0 += kc) {
    const int buf = consumed % kNBuf;
    mbar_wait(&ch.st->full[buf], (consumed / kNBuf) & 1, &ch.st->abort_flag);
    const int rows = min(kc, K - k0);
    const int per = rows / ksplit;  // rows of this slab handled by one k-group
    if (active) {
      int wo = buf * (kBufBytes / 4) + (kg * per) * N + cg;  // ring lives at offset 0
      int ao = a_off + k0 + kg * per;
#pragma unroll 2
      for (int k = 0; k < per; k += 4) {
        float w[CPT][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int c = 0; c < CPT; ++c) w[c][i] = g_smem[wo + i * N + c * cols];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const float4 a = *reinterpret_cast<const float4*>(&g_smem[ao + r * lda]);
#pragma unroll
          for (int c = 0; c < CPT; ++c) {
            acc[c][r] = fmaf(a.x, w[c][0], acc[c][r]);
            acc[c][r] = fmaf(a.y, w[c][1], acc[c][r]);
            acc[c][r] = fmaf(a.z, w[c][2], acc[c][r]);
            acc[c][r] = fmaf(a.w, w[c][3], acc[c][r]);
          }
        }
        wo += 4 * N;
        ao += 4;
      }
    }
    ++consumed;
    __syncwarp();
    if ((threadIdx.x & 31) == 0)  // this warp is done with the ring slot
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&ch.st->empty[buf])) : "memory");
  }
  ch.consumed = consumed;

  // k-groups 1.. park their partial sums; group 0 adds them in a fixed order
  if (ksplit > 1) {
    if (active && kg > 0) {
#pragma unroll
      for (int c = 0; c < CPT; ++c)
#pragma unroll
        for (int r = 0; r < R; ++r) g_smem[ch.scratch + ((kg - 1) * R + r) * N + cg + c * cols] = acc[c][r];
    }
    sync_compute(ch.T);
  }
  if (active && kg == 0) {
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      const int n = cg + c * cols;
      const float b = bias ? __ldg(bias + n) : 0.f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float v = acc[c][r];
        for (int kk = 1; kk < ksplit; ++kk) v += g_smem[ch.scratch + ((kk - 1) * R + r) * N + n];
        v += b;
        if (gelu) v = gelu_erf(v);
        g_smem[o_off + r * ldo + n] = v;
      }
    }
  }
  sync_compute(ch.T);
}

template <int R>
__device__ __forceinline__ void gemm_rows(Chain& ch, int K, int N, const float* s_a, int lda,
                                          const float* __restrict__ bias, bool gelu, float* s_o, int ldo) {
  const int a_off = (int)(s_a - g_smem), o_off = (int)(s_o - g_smem);
  int cpt, ksplit;
  plan_gemm(K, N, ch.T, ch.cap, cpt, ksplit);
  switch (cpt) {
    case 4: gemm_body<R, 4>(ch, K, N, ksplit, a_off, lda, bias, gelu, o_off, ldo); break;
    case 3: gemm_body<R, 3>(ch, K, N, ksplit, a_off, lda, bias, gelu, o_off, ldo); break;
    case 2: gemm_body<R, 2>(ch, K, N, ksplit, a_off, lda, bias, gelu, o_off, ldo); break;
    default: gemm_body<R, 1>(ch, K, N, ksplit, a_off, lda, bias, gelu, o_off, ldo); break;
  }
}

// dst[r][:] = LayerNorm(a[r][:] + b[r][:]) * gamma + beta   (b optional; a, b, dst may alias row-wise)
template <int R>
__device__ __forceinline__ void ln_rows(float* dst, int ldd, const float* a, int lda, const float* b, int ldb,
                                        const float* __restrict__ gamma, const float* __restrict__ beta, int D,
                                        int n_valid, int T) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = T >> 5;
  for (int r = warp; r < R; r += nw) {
    if (r >= n_valid) continue;
    float s = 0.f;
    for (int d = lane; d < D; d += 32) {
      float v = a[r * lda + d];
      if (b) v += b[(size_t)r * ldb + d];
      s += v;
    }
    const float mean = warp_sum(s) / (float)D;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
      float v = a[r * lda + d];
      if (b) v += b[(size_t)r * ldb + d];
      v -= mean;
      ss = fmaf(v, v, ss);
    }
    const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)D + 1e-5f);
    for (int d = lane; d < D; d += 32) {
      float v = a[r * lda + d];
      if (b) v += b[(size_t)r * ldb + d];
      dst[r * ldd + d] = (v - mean) * rstd * __ldg(gamma + d) + __ldg(beta + d);
    }
  }
  sync_compute(T);
}

// One warp per head row: mixture parameters from raw[3K], then sample or log-pdf.
__device__ __forceinline__ void head_row(const DenseArgs& a, const float* raw, long row) {
  const int lane = threadIdx.x & 31;
  const int K = a.n_comp;
  const long b = row / a.head_tps;
  const int j = (int)(row - b * a.head_tps);
  if (j < a.head_first) return;
  const long oidx = b * a.out_stride + a.out_col + (j - a.head_first);
  float mean = 0.f, stdv = 1.f, lw = -INFINITY;
  if (lane < K) {
    mean = raw[3 * lane] + __ldg(a.mean_bias + lane);
    const float sr = raw[3 * lane + 1] + __ldg(a.std_bias + lane);
    const float sp = sr > 20.f ? sr : log1pf(expf(sr));  // F.softplus, beta 1, threshold 20
    stdv = fminf(sp, 2.0f) + 1e-3f;
    lw = raw[3 * lane + 2] + __ldg(a.weight_bias + lane);
  }
  const float mx = warp_max(lw);
  const float se = warp_sum(lane < K ? expf(lw - mx) : 0.f);
  const float logw = lw - mx - logf(se);  // log_softmax
  float y;
  if (a.head_mode == 1) {
    // torch.multinomial(w, 1) == argmax_k(w_k / Exp(1)_k); first maximum wins
    float ratio = -1.f;
    if (lane < K) ratio = expf(logw) / __ldg(a.expo + b * K + lane);
    int best = lane;
    float bv = ratio;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best, o);
      if (ov > bv || (ov == bv && oi < best)) {
        bv = ov;
        best = oi;
      }
    }
    const float m_sel = __shfl_sync(0xffffffffu, mean, best);
    const float s_sel = __shfl_sync(0xffffffffu, stdv, best);
    y = m_sel + s_sel * __ldg(a.normal + b);
    if (lane == 0) {
      a.y_out[oidx] = y;
      if (a.comp_out) a.comp_out[oidx] = best;
    }
  } else {
    y = __ldg(a.y_in + oidx);
  }
  if (a.ld_out) {
    float lp = -INFINITY;
    if (lane < K) {
      const float zz = (y - mean) / stdv;
      lp = -0.5f * (1.8378770664093453f + 2.0f * logf(stdv) + zz * zz) + logw;
    }
    const float m2 = warp_max(lp);
    const float s2 = warp_sum(lane < K ? expf(lp - m2) : 0.f);
    if (lane == 0) a.ld_out[oidx] = m2 + logf(s2);
  }
}

template <int R>
__global__ void __launch_bounds__(288) dense_chain_kernel(const DenseArgs a) {
  float* const smem = g_smem;
  const int D = a.D, Dff = a.Dff;
  const int wide = max(3 * D, Dff);
  const int T = blockDim.x - 32;                    // compute threads; the last warp streams weights
  float* ring = smem;                               // weight ring
  float* s_x = ring + kNBuf * (kBufBytes / 4);      // [R][D]
  float* s_t = s_x + R * D;                         // [R][D]
  float* s_h = s_t + R * D;                         // [R][wide]
  float* scratch = s_h + R * wide;                  // [3][R][D]
  Stream* st = reinterpret_cast<Stream*>(scratch + 3 * R * D);
  const long row0 = (long)blockIdx.x * R;
  const int n_valid = (int)min((long)R, (long)a.rows - row0);

  if (threadIdx.x == 0) {
    st->abort_flag = 0;
    for (int i = 0; i < kNBuf; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&st->full[i])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&st->empty[i])), "r"(T >> 5) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if ((int)threadIdx.x >= T) {
    // ------------------------------ producer warp ------------------------------
    if (threadIdx.x == T) {
      int issued = 0;
      bool ok = true;
      if (a.do_post) {
        ok = ok && produce(st, ring, issued, a.post_w.wo_t, D, D, T, 3 * D);
        ok = ok && produce(st, ring, issued, a.post_w.w1_t, D, Dff, T, 3 * D);
        ok = ok && produce(st, ring, issued, a.post_w.w2_t, Dff, D, T, 3 * D);
      }
      if (a.do_head) {
        ok = ok && produce(st, ring, issued, a.wa_t, D, Dff, T, 3 * D);
        ok = ok && produce(st, ring, issued, a.wb_t, Dff, 3 * a.n_comp, T, 3 * D);
      } else if (a.do_pre) {
        ok = ok && produce(st, ring, issued, a.pre_w.wf_t, D, D, T, 3 * D);
        ok = ok && produce(st, ring, issued, a.pre_w.wqkv_t, D, 3 * D, T, 3 * D);
      }
    }
    return;
  }

  Chain ch;
  ch.st = st;
  ch.scratch = (int)(scratch - g_smem);
  ch.consumed = 0;
  ch.T = T;
  ch.cap = 3 * D;
  float* cur = s_x;

  if (a.do_post) {
    // s_h[0..R*D) <- attention output rows
    for (int i = threadIdx.x; i < R * D; i += T) {
      const int r = i / D;
      s_h[i] = r < n_valid ? a.attn[(size_t)row0 * D + i] : 0.f;
    }
    sync_compute(T);
    gemm_rows<R>(ch, D, D, s_h, D, nullptr, false, s_t, D);
    ln_rows<R>(s_x, D, s_t, D, a.x1_in + (size_t)row0 * D, D, a.post_w.ln2_g, a.post_w.ln2_b, D, n_valid, T);
    gemm_rows<R>(ch, D, Dff, s_x, D, a.post_w.b1, true, s_h, wide);
    gemm_rows<R>(ch, Dff, D, s_h, wide, a.post_w.b2, false, s_t, D);
    ln_rows<R>(s_x, D, s_x, D, s_t, D, a.post_w.ln3_g, a.post_w.ln3_b, D, n_valid, T);
    if (a.x_out) {
      for (int i = threadIdx.x; i < n_valid * D; i += T) a.x_out[(size_t)row0 * D + i] = s_x[i];
    }
  } else {
    for (int i = threadIdx.x; i < R * D; i += T) {
      const int r = i / D;
      s_x[i] = r < n_valid ? a.x_in[(size_t)row0 * D + i] : 0.f;
    }
    sync_compute(T);
  }

  if (a.do_final) {
    ln_rows<R>(s_t, D, s_x, D, nullptr, 0, a.lnf_g, a.lnf_b, D, n_valid, T);
    cur = s_t;
    if (a.z_out) {
      for (int i = threadIdx.x; i < n_valid * D; i += T) a.z_out[(size_t)row0 * D + i] = s_t[i];
    }
  }

  if (a.do_head) {
    float* s_raw = (cur == s_x) ? s_t : s_x;
    gemm_rows<R>(ch, D, Dff, cur, D, a.ba, true, s_h, wide);
    gemm_rows<R>(ch, Dff, 3 * a.n_comp, s_h, wide, a.bb, false, s_raw, D);
    if (!st->abort_flag) {
      const int warp = threadIdx.x >> 5, nw = T >> 5;
      for (int r = warp; r < n_valid; r += nw) head_row(a, s_raw + r * D, row0 + r);
    }
  } else if (a.do_pre) {
    // feature attention over one token == out_proj(v_proj(x)); folded into wf_t
    gemm_rows<R>(ch, D, D, s_x, D, nullptr, false, s_t, D);
    ln_rows<R>(s_x, D, s_x, D, s_t, D, a.pre_w.ln1_g, a.pre_w.ln1_b, D, n_valid, T);
    for (int i = threadIdx.x; i < n_valid * D; i += T) a.x1_out[(size_t)row0 * D + i] = s_x[i];
    gemm_rows<R>(ch, D, 3 * D, s_x, D, nullptr, false, s_h, wide);
    const bool bf = a.kv.dtype == ARTAB_BF16;
    for (int i = threadIdx.x; i < n_valid * D; i += T) {
      const int r = i / D, c = i - r * D;
      const float qv = s_h[r * wide + c];
      if (bf)
        reinterpret_cast<__nv_bfloat16*>(a.q_out)[(size_t)row0 * D + i] = __float2bfloat16_rn(qv);
      else
        reinterpret_cast<float*>(a.q_out)[(size_t)row0 * D + i] = qv;
      if (a.kv.mode != KV_NONE) {
        const float kv_k = s_h[r * wide + D + c], kv_v = s_h[r * wide + 2 * D + c];
        if (bf) {
          scatter_k<__nv_bfloat16>(a.kv, row0 + r, c, kv_k);
          scatter_v<__nv_bfloat16>(a.kv, row0 + r, c, kv_v);
        } else {
          scatter_k<float>(a.kv, row0 + r, c, kv_k);
          scatter_v<float>(a.kv, row0 + r, c, kv_v);
        }
      }
    }
  }
  if (threadIdx.x == 0 && st->abort_flag && a.status) atomicExch(a.status, 2);
}

__global__ void __launch_bounds__(128) embed_kernel(const EmbedArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (threadIdx.x == 0) ARTAB_STAMP(0, 0);
  dep_wait();
  dep_trigger();
  if (threadIdx.x == 0) ARTAB_STAMP(0, 1);
  if (row >= a.rows) return;
  const float* xr;
  float yv = 0.f;
  bool has_y = false;
  int kind = a.kind, ar = -1;
  if (a.mode == EMB_ROWS) {
    xr = a.x + (size_t)row * a.F;
    if (a.y) {
      yv = a.y[row];
      has_y = true;
    }
    if (a.ar_idx) ar = a.ar_idx[row];
  } else if (a.mode == EMB_DECODE) {
    // step t: [buffer(x_{t-1}, y_{t-1}, ar = t mod S), target(x_t)]; t = 0: target only
    const long b = row / a.n_new;
    const int j = (int)(row - b * a.n_new);
    if (a.n_new == 2 && j == 0) {
      xr = a.xt + ((size_t)b * a.Nt + (a.t - 1)) * a.F;
      yv = a.yt[(size_t)b * a.Nt + (a.t - 1)];
      has_y = true;
      kind = ARTAB_MARK_BUFFER;
      ar = a.t % a.S;
    } else {
      xr = a.xt + ((size_t)b * a.Nt + a.t) * a.F;
      kind = ARTAB_MARK_TARGET;
    }
  } else if (a.mode == EMB_FWD) {
    // masked forward: [Buffer_0..Buffer_{Nb-1}, Target_0..Target_{Nt-1}], buffer j carries ar = j (Nb <= S)
    const int tps = a.Nb + a.Nt;
    const long b = row / tps;
    const int j = (int)(row - b * tps);
    if (j < a.Nb) {
      xr = a.xb + ((size_t)b * a.Nb + j) * a.F;
      yv = a.yb[(size_t)b * a.Nb + j];
      has_y = true;
      kind = ARTAB_MARK_BUFFER;
      ar = j;
    } else {
      xr = a.xt + ((size_t)b * a.Nt + (j - a.Nb)) * a.F;
      kind = ARTAB_MARK_TARGET;
    }
  } else {
    // teacher forcing: [Buffer_0..Buffer_{Nt-1}, Target_0..Target_{Nt-1}], buffer j carries ar = j mod S
    const long b = row / (2 * a.Nt);
    const int j = (int)(row - b * 2 * a.Nt);
    if (j < a.Nt) {
      xr = a.xt + ((size_t)b * a.Nt + j) * a.F;
      yv = a.yt[(size_t)b * a.Nt + j];
      has_y = true;
      kind = ARTAB_MARK_BUFFER;
      ar = j % a.S;
    } else {
      xr = a.xt + ((size_t)b * a.Nt + (j - a.Nt)) * a.F;
      kind = ARTAB_MARK_TARGET;
    }
  }
  float s = 0.f;
  for (int f = lane; f < a.F; f += 32) s += xr[f];
  const float xm = warp_sum(s) / (float)a.F;
  for (int d = lane; d < a.D; d += 32) {
    float e = fmaf(xm, __ldg(a.wx + d), __ldg(a.bx + d));
    if (has_y) e += fmaf(yv, __ldg(a.wy + d), __ldg(a.by + d));
    e += __ldg(a.marker + kind * a.D + d);
    if (ar >= 0) e += __ldg(a.ar_tokens + ar * a.D + d);
    a.out[a.out_lane_major ? lane_major_index(row, d, a.D) : (size_t)row * a.D + d] = e;
  }
}

}  // namespace

int launch_embed(const EmbedArgs& a, cudaStream_t s) {
  if (a.rows <= 0) return ARTAB_OK;
  const int wpb = 4;
  prof_begin(PROF_EMBED, s);
  ARTAB_STAMP_ATTACH();
  const cudaError_t le = launch_dependent(embed_kernel, dim3((unsigned)((a.rows + wpb - 1) / wpb)), dim3(wpb * 32), 0, s, a);
  prof_end(s);
  ARTAB_REQUIRE(le == cudaSuccess, ARTAB_ELAUNCH, "embed_kernel: %s", cudaGetErrorString(le));
  count_launch();
  return check_launch("embed_kernel");
}

int launch_dense(const DenseArgs& a, cudaStream_t s) {
  if (a.rows <= 0) return ARTAB_OK;
  if (dense_tc_applicable(a)) return launch_dense_tc(a, s);
  ARTAB_REQUIRE(a.D % 32 == 0 && a.Dff % 4 == 0 && a.D >= 32, ARTAB_EINVAL,
                "dense chain: d_model must be a multiple of 32 and d_ff a multiple of 4 (got %d, %d)", a.D, a.Dff);
  ARTAB_REQUIRE(3 * a.n_comp <= a.D && a.n_comp <= 32, ARTAB_EINVAL, "dense chain: need 3*K <= d_model and K <= 32");
  ARTAB_REQUIRE(a.D % 16 == 0 && a.Dff % 16 == 0, ARTAB_EINVAL, "dense chain: d_model and d_ff must be multiples of 16");
  // compute threads: d_model of them (at most 256), more when a wider GEMM needs them to cover its
  // columns at four per thread
  int T = 0;
  for (int t = a.D <= 256 ? a.D : 256; t <= 256 && !T; t += 32) {
    const int cap = 3 * a.D;
    // (K, N) of every GEMM of the chain: Wo / Wf, W1 / head.0, W2, Wq|Wk|Wv, head.2
    if (gemm_plan_ok(a.D, a.D, t, cap) && gemm_plan_ok(a.D, a.Dff, t, cap) && gemm_plan_ok(a.Dff, a.D, t, cap) &&
        gemm_plan_ok(a.D, 3 * a.D, t, cap) && gemm_plan_ok(a.Dff, 3 * a.n_comp, t, cap))
      T = t;
  }
  ARTAB_REQUIRE(T > 0, ARTAB_EINVAL, "dense chain: no thread plan for d_model %d, d_ff %d (d_ff at most 1024)", a.D,
                a.Dff);
  const int wide = 3 * a.D > a.Dff ? 3 * a.D : a.Dff;
  const size_t smem = (size_t)kNBuf * kBufBytes + (size_t)kRows * (2 * a.D + wide + 3 * a.D) * sizeof(float) +
                      sizeof(Stream) + 128;
  static SmemConfig configured;
  {
    const cudaError_t e = configured.ensure(dense_chain_kernel<kRows>, smem);
    ARTAB_REQUIRE(e == cudaSuccess, ARTAB_ELAUNCH, "dense chain: %zu bytes of shared memory refused: %s", smem,
                  cudaGetErrorString(e));
  }
  const int threads = T + 32;  // compute threads + the weight-streaming warp
  const int grid = (a.rows + kRows - 1) / kRows;
  prof_begin(PROF_DENSE, s);
  dense_chain_kernel<kRows><<<grid, threads, smem, s>>>(a);
  prof_end(s);
  count_launch();
  return check_launch("dense_chain_kernel");
}

}  // namespace artab
