// SIMT attention kernels.
//
//  * ctx_attn_simt_kernel  — queries of many streams against one shared (or one
//    per-group) context K/V with online softmax and LSE output; fp32 FMA math.
//    This is the context kernel of the fp32 mode (and of head sizes the
//    tensor-core kernel is not built for).
//  * buf_merge_kernel      — the bandwidth-bound warp-level pass over each
//    stream's private buffer K/V, merged in registers by log-sum-exp with the
//    context partials (any number of key splits).  Used by both dtypes.
//  * kv_append_kernel      — in-place append of one K/V row per (stream, head).
#include "attn.cuh"

namespace artab {

namespace {

constexpr int kQW = 4;        // queries per warp
constexpr int kWarps = 4;     // warps per CTA
constexpr int kQB = kQW * kWarps;
constexpr int kKT = 64;       // keys per tile

template <typename T, int DH>
__global__ void __launch_bounds__(kWarps * 32) ctx_attn_simt_kernel(const CtxAttnArgs a) {
  constexpr int NDL = DH >= 32 ? DH / 32 : 1;  // output dims per lane
  __shared__ float sK[kKT][DH + 1];
  __shared__ float sV[kKT][DH];
  __shared__ float sQ[kQB][DH];
  __shared__ __align__(16) float sP[kWarps][kKT][kQW];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int g = blockIdx.z / a.n_splits, split = blockIdx.z - g * a.n_splits;
  const int rows_in_group = a.n_groups == 1 ? a.rows : a.rows_per_group;
  const long group_row0 = a.n_groups == 1 ? 0 : (long)g * a.rows_per_group;
  const int q0 = blockIdx.x * kQB;
  if (q0 >= rows_in_group) return;

  const int tiles = (a.n_ctx + kKT - 1) / kKT;
  const int tps = (tiles + a.n_splits - 1) / a.n_splits;
  const int k_begin = split * tps * kKT;
  const int k_end = min(a.n_ctx, k_begin + tps * kKT);

  const T* Q = reinterpret_cast<const T*>(a.q);
  const T* Kc = reinterpret_cast<const T*>(a.k_ctx) + ((size_t)(g * a.n_heads + h) * a.n_ctx_pad) * DH;
  // transposed layout holds a hi and a lo part per head: [2*Dh][Ncp]
  const T* Vc = reinterpret_cast<const T*>(a.v_ctx) +
                ((size_t)(g * a.n_heads + h) * a.n_ctx_pad) * DH * (a.v_transposed ? 2 : 1);

  for (int i = threadIdx.x; i < kQB * DH; i += blockDim.x) {
    const int qi = i / DH, d = i - qi * DH;
    const int r = q0 + qi;
    sQ[qi][d] = r < rows_in_group ? to_f32<T>(Q[((size_t)(group_row0 + r) * a.n_heads + h) * DH + d]) : 0.f;
  }

  float m[kQW], l[kQW], acc[kQW][NDL];
#pragma unroll
  for (int qq = 0; qq < kQW; ++qq) {
    m[qq] = -INFINITY;
    l[qq] = 0.f;
#pragma unroll
    for (int e = 0; e < NDL; ++e) acc[qq][e] = 0.f;
  }
  const float sc = a.scale * kLog2e;

  for (int kt = k_begin; kt < k_end; kt += kKT) {
    __syncthreads();
    for (int i = threadIdx.x; i < kKT * DH; i += blockDim.x) {
      const int key = i / DH, d = i - key * DH;
      sK[key][d] = (kt + key) < a.n_ctx ? to_f32<T>(Kc[(size_t)(kt + key) * DH + d]) : 0.f;
    }
    if (a.v_transposed) {
      for (int i = threadIdx.x; i < kKT * DH; i += blockDim.x) {
        const int d = i / kKT, key = i - d * kKT;
        sV[key][d] = (kt + key) < a.n_ctx ? to_f32<T>(Vc[(size_t)d * a.n_ctx_pad + kt + key]) +
                                                 to_f32<T>(Vc[(size_t)(DH + d) * a.n_ctx_pad + kt + key])
                                           : 0.f;
      }
    } else {
      for (int i = threadIdx.x; i < kKT * DH; i += blockDim.x) {
        const int key = i / DH, d = i - key * DH;
        sV[key][d] = (kt + key) < a.n_ctx ? to_f32<T>(Vc[(size_t)(kt + key) * DH + d]) : 0.f;
      }
    }
    __syncthreads();

    float s0[kQW], s1[kQW];
#pragma unroll
    for (int qq = 0; qq < kQW; ++qq) s0[qq] = s1[qq] = 0.f;
#pragma unroll 8
    for (int d = 0; d < DH; ++d) {
      const float k0 = sK[lane][d], k1 = sK[lane + 32][d];
#pragma unroll
      for (int qq = 0; qq < kQW; ++qq) {
        const float qv = sQ[warp * kQW + qq][d];
        s0[qq] = fmaf(qv, k0, s0[qq]);
        s1[qq] = fmaf(qv, k1, s1[qq]);
      }
    }
    const bool v0 = kt + lane < k_end, v1 = kt + lane + 32 < k_end;
#pragma unroll
    for (int qq = 0; qq < kQW; ++qq) {
      const float a0 = v0 ? s0[qq] * sc : -INFINITY;
      const float a1 = v1 ? s1[qq] * sc : -INFINITY;
      const float mn = fmaxf(m[qq], warp_max(fmaxf(a0, a1)));  // finite: every tile holds a valid key
      const float alpha = exp2f(m[qq] - mn);
      const float p0 = exp2f(a0 - mn), p1 = exp2f(a1 - mn);
      l[qq] = l[qq] * alpha + warp_sum(p0 + p1);
      m[qq] = mn;
#pragma unroll
      for (int e = 0; e < NDL; ++e) acc[qq][e] *= alpha;
      sP[warp][lane][qq] = p0;
      sP[warp][lane + 32][qq] = p1;
    }
    __syncwarp();
    if (DH >= 32 || lane < DH) {
#pragma unroll 4
      for (int key = 0; key < kKT; ++key) {
        const float4 p4 = *reinterpret_cast<const float4*>(&sP[warp][key][0]);
#pragma unroll
        for (int e = 0; e < NDL; ++e) {
          const float v = sV[key][lane + 32 * e];
          acc[0][e] = fmaf(p4.x, v, acc[0][e]);
          acc[1][e] = fmaf(p4.y, v, acc[1][e]);
          acc[2][e] = fmaf(p4.z, v, acc[2][e]);
          acc[3][e] = fmaf(p4.w, v, acc[3][e]);
        }
      }
    }
    __syncwarp();
  }

#pragma unroll
  for (int qq = 0; qq < kQW; ++qq) {
    const int r = q0 + warp * kQW + qq;
    if (r >= rows_in_group) continue;
    const size_t ro = ((size_t)split * a.rows + group_row0 + r) * a.n_heads + h;
    const float inv = l[qq] > 0.f ? 1.0f / l[qq] : 0.f;
    if (DH >= 32 || lane < DH) {
#pragma unroll
      for (int e = 0; e < NDL; ++e) {
        const size_t idx = a.out_lane_major
                               ? lane_major_index(group_row0 + r, h * DH + lane + 32 * e, a.n_heads * DH)
                               : ro * DH + lane + 32 * e;
        a.out[idx] = acc[qq][e] * inv;
      }
    }
    if (lane == 0) a.lse[ro] = l[qq] > 0.f ? (m[qq] + log2f(l[qq])) * kLn2 : -INFINITY;
  }
}

__device__ __forceinline__ float fast_exp2(float x) {  // MUFU ex2: relative error 2^-22, exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------
// Private-buffer pass + merge.  One warp per (stream, head[, item]).
// Each key's K row and V row are adjacent in memory ([.., T][2][Dh]), so a warp
// iteration reads one contiguous span of KPI keys; LPK lanes share a key, each
// holding one 16-byte slice of the K row and of the V row.
// ---------------------------------------------------------------------------
template <typename T, int DH>
__global__ void __launch_bounds__(128, 6) buf_merge_kernel(const BufMergeArgs a) {
  dep_trigger();  // the dependent dense chain reads only model constants before its wait (see buf_mma_kernel)
  constexpr int VEC = Vec16<T>::N;
  constexpr int LPK = DH / VEC;   // lanes per key
  constexpr int KPI = 32 / LPK;   // keys per warp iteration
  static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "head_dim must give a power-of-two slice count");
  const int lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= a.n_items) return;
  const int sub = lane % LPK, grp = lane / LPK;

  long b;
  int h, len;
  long row_t, row_b;
  const uint8_t* mrow = nullptr;  // optional per-key visibility of this item's query (mode 2)
  if (a.mode_tf == 2) {
    // one query per item: token j of stream b sees the first visible[j] buffer rows
    const int j = (int)(item % a.tps);
    const long bh = item / a.tps;
    b = bh / a.n_heads;
    h = (int)(bh - b * a.n_heads);
    len = min(max(__ldg(a.visible + j), 0), a.len0);  // len0: buffer rows written per stream
    row_t = b * a.tps + j;
    row_b = -1;
    if (a.key_mask) mrow = a.key_mask + ((size_t)row_t * a.n_heads + h) * a.max_buf;
  } else if (a.mode_tf) {
    const int ips = a.nt + 1;
    const int i = (int)(item % ips);
    const long bh = item / ips;
    b = bh / a.n_heads;
    h = (int)(bh - b * a.n_heads);
    len = i;
    row_t = i < a.nt ? b * 2 * a.nt + a.nt + i : -1;
    row_b = i >= 1 ? b * 2 * a.nt + i - 1 : -1;
  } else {
    b = item / a.n_heads;
    h = (int)(item - b * a.n_heads);
    len = a.lens ? min(max(__ldg(a.lens + b), 0), a.len0) : a.len0;
    row_t = b * a.n_new + a.n_new - 1;
    row_b = a.n_new == 2 ? b * a.n_new : -1;
  }

  const T* Q = reinterpret_cast<const T*>(a.q);
  const float sc = a.scale * kLog2e;
  float q[2][VEC];
  const long rows2[2] = {row_t, row_b};
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    if (rows2[w] >= 0) {
      Vec16<T>::load(Q + ((size_t)rows2[w] * a.n_heads + h) * DH + sub * VEC, q[w]);
#pragma unroll
      for (int e = 0; e < VEC; ++e) q[w][e] *= sc;
    } else {
#pragma unroll
      for (int e = 0; e < VEC; ++e) q[w][e] = 0.f;
    }
  }

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f}, acc[2][VEC];
#pragma unroll
  for (int w = 0; w < 2; ++w)
#pragma unroll
    for (int e = 0; e < VEC; ++e) acc[w][e] = 0.f;

  const T* kv = reinterpret_cast<const T*>(a.kv_buf) + ((size_t)(b * a.n_heads + h) * a.max_buf) * 2 * DH;
  // Keys are walked in chunks of CH warp iterations: all 2*CH 16-byte loads of a chunk are issued
  // before the first is used, so a warp has CH KiB in flight and pays one memory round trip per
  // chunk instead of one per iteration.
  constexpr int CH = 4;
  for (int key0 = 0; key0 < len; key0 += KPI * CH) {
    uint4 kr[CH], vr[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int key = key0 + c * KPI + grp;
      if (key < len) {
        const uint4* p = reinterpret_cast<const uint4*>(kv + (size_t)key * 2 * DH + sub * VEC);
        kr[c] = __ldg(p);
        vr[c] = __ldg(p + LPK);  // the V row follows the K row: DH elements = LPK 16-byte slices
      } else {
        kr[c] = make_uint4(0u, 0u, 0u, 0u);
        vr[c] = kr[c];
      }
    }
    // scores of the chunk first, then ONE running-max update and rescale for all CH keys
    float sc0[CH], sc1[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      sc0[c] = sc1[c] = -INFINITY;
      if (key0 + c * KPI >= len) continue;  // warp-uniform: a short tail skips the empty iterations
      float kf[VEC];
      Vec16<T>::unpack(kr[c], kf);
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        s0 = fmaf(q[0][e], kf[e], s0);
        s1 = fmaf(q[1][e], kf[e], s1);
      }
#pragma unroll
      for (int o = 1; o < LPK; o <<= 1) {
        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
      }
      bool valid = key0 + c * KPI + grp < len;
      if (valid && mrow) valid = mrow[key0 + c * KPI + grp] != 0;
      sc0[c] = valid ? s0 : -INFINITY;
      sc1[c] = valid ? s1 : -INFINITY;
    }
    if (key0 + grp < len) {  // this lane group has at least one key in the chunk
      float mn0 = m[0], mn1 = m[1];
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        mn0 = fmaxf(mn0, sc0[c]);
        mn1 = fmaxf(mn1, sc1[c]);
      }
      // a lane group whose keys are all masked so far keeps mn = -inf: nothing to rescale, and its
      // exponentials below are taken against 0 instead (exp2(-inf - 0) = 0 for the masked keys)
      const float a0 = mn0 == -INFINITY ? 1.0f : fast_exp2(m[0] - mn0);
      const float a1 = mn1 == -INFINITY ? 1.0f : fast_exp2(m[1] - mn1);
      const float r0 = mn0 == -INFINITY ? 0.0f : mn0, r1 = mn1 == -INFINITY ? 0.0f : mn1;
      l[0] *= a0;
      l[1] *= a1;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        acc[0][e] *= a0;
        acc[1][e] *= a1;
      }
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        if (key0 + c * KPI >= len) continue;
        float vf[VEC];
        Vec16<T>::unpack(vr[c], vf);
        const float p0 = fast_exp2(sc0[c] - r0), p1 = fast_exp2(sc1[c] - r1);  // masked keys: exp2(-inf) = 0
        l[0] += p0;
        l[1] += p1;
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          acc[0][e] = fmaf(p0, vf[e], acc[0][e]);
          acc[1][e] = fmaf(p1, vf[e], acc[1][e]);
        }
      }
      m[0] = mn0;
      m[1] = mn1;
    }
  }
  // fold the KPI per-group partial softmaxes together
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
    for (int w = 0; w < 2; ++w) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[w], o);
      const float lo = __shfl_xor_sync(0xffffffffu, l[w], o);
      const float mn = fmaxf(m[w], mo);
      const float a1 = mn == -INFINITY ? 0.f : fast_exp2(m[w] - mn);
      const float a2 = mn == -INFINITY ? 0.f : fast_exp2(mo - mn);
      l[w] = l[w] * a1 + lo * a2;
      m[w] = mn;
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[w][e], o);
        acc[w][e] = acc[w][e] * a1 + ao * a2;
      }
    }
  }

  // The buffer pass above read only what kernels older than the preceding one wrote (q and the
  // buffer rows); the context partials come from the preceding kernel.
  dep_wait();

  // log-sum-exp merge with the context partials, all in registers
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    const long r = rows2[w];
    if (r < 0) continue;
    float lse_b = l[w] > 0.f ? (m[w] + log2f(l[w])) * kLn2 : -INFINITY;  // natural log, like the partials
    float top = lse_b;
    for (int s = 0; s < a.n_splits; ++s)
      top = fmaxf(top, __ldg(a.lse_part + ((size_t)s * a.rows + r) * a.n_heads + h));
    float wsum = 0.f, o[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) o[e] = 0.f;
    if (l[w] > 0.f) {
      const float wb = expf(lse_b - top);
      wsum = wb;
      const float inv = wb / l[w];
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] = acc[w][e] * inv;
    }
    for (int s = 0; s < a.n_splits; ++s) {
      const size_t ro = ((size_t)s * a.rows + r) * a.n_heads + h;
      const float ls = __ldg(a.lse_part + ro);
      if (ls == -INFINITY) continue;
      const float ws = expf(ls - top);
      wsum += ws;
      const float* op = a.o_part + ro * DH + sub * VEC;
#pragma unroll
      for (int e = 0; e < VEC; e += 4) {
        const float4 v = *reinterpret_cast<const float4*>(op + e);
        o[e] = fmaf(ws, v.x, o[e]);
        o[e + 1] = fmaf(ws, v.y, o[e + 1]);
        o[e + 2] = fmaf(ws, v.z, o[e + 2]);
        o[e + 3] = fmaf(ws, v.w, o[e + 3]);
      }
    }
    if (a.lse_out && lane == 0) a.lse_out[(size_t)r * a.n_heads + h] = wsum > 0.f ? top + logf(wsum) : -INFINITY;
    if (grp == 0) {
      float inv = wsum > 0.f ? 1.0f / wsum : 0.f;
      if (a.poison_if && __ldcg(a.poison_if) != 0) inv = __int_as_float(0x7fc00000);
#pragma unroll
      for (int e = 0; e < VEC; e += 4) {
        float* dst = a.out + (a.out_lane_major ? lane_major_index(r, h * DH + sub * VEC + e, a.n_heads * DH)
                                               : ((size_t)r * a.n_heads + h) * DH + sub * VEC + e);
        *reinterpret_cast<float4*>(dst) = make_float4(o[e] * inv, o[e + 1] * inv, o[e + 2] * inv, o[e + 3] * inv);
      }
    }
  }
}

template <typename T>
__global__ void kv_append_kernel(T* kv, const T* k_new, const T* v_new, long n_bh, int dh, int max_buf, int pos) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_bh * dh) return;
  const long bh = i / dh;
  const int d = (int)(i - bh * dh);
  T* p = kv + ((size_t)bh * max_buf + pos) * 2 * dh + d;
  p[0] = k_new[i];
  p[dh] = v_new[i];
}

template <typename T>
int launch_ctx_t(const CtxAttnArgs& a, cudaStream_t s) {
  const int rows_in_group = a.n_groups == 1 ? a.rows : a.rows_per_group;
  dim3 grid((rows_in_group + kQB - 1) / kQB, a.n_heads, a.n_groups * a.n_splits);
  ARTAB_REQUIRE(a.head_dim == 16 || a.head_dim == 32 || a.head_dim == 64, ARTAB_EINVAL,
                "context attention: head_dim %d not supported (16, 32, 64)", a.head_dim);
  prof_begin(PROF_CTX, s);
  switch (a.head_dim) {
    case 16: ctx_attn_simt_kernel<T, 16><<<grid, kWarps * 32, 0, s>>>(a); break;
    case 32: ctx_attn_simt_kernel<T, 32><<<grid, kWarps * 32, 0, s>>>(a); break;
    default: ctx_attn_simt_kernel<T, 64><<<grid, kWarps * 32, 0, s>>>(a); break;
  }
  prof_end(s);
  count_launch();
  return check_launch("ctx_attn_simt_kernel");
}

template <typename T>
int launch_buf_t(const BufMergeArgs& a, cudaStream_t s) {
  const int wpb = 4;
  const unsigned grid = (unsigned)((a.n_items + wpb - 1) / wpb);
  cudaError_t le = cudaSuccess;
  ARTAB_REQUIRE(a.head_dim == 16 || a.head_dim == 32 || a.head_dim == 64, ARTAB_EINVAL,
                "buffer attention: head_dim %d not supported (16, 32, 64)", a.head_dim);
  prof_begin(PROF_BUF, s);
  switch (a.head_dim) {
    case 16: le = launch_dependent(buf_merge_kernel<T, 16>, dim3(grid), dim3(wpb * 32), 0, s, a); break;
    case 32: le = launch_dependent(buf_merge_kernel<T, 32>, dim3(grid), dim3(wpb * 32), 0, s, a); break;
    default: le = launch_dependent(buf_merge_kernel<T, 64>, dim3(grid), dim3(wpb * 32), 0, s, a); break;
  }
  prof_end(s);
  ARTAB_REQUIRE(le == cudaSuccess, ARTAB_ELAUNCH, "buf_merge_kernel: %s", cudaGetErrorString(le));
  count_launch();
  return check_launch("buf_merge_kernel");
}

}  // namespace

int launch_ctx_attn_simt(const CtxAttnArgs& a, cudaStream_t s) {
  if (a.rows <= 0) return ARTAB_OK;
  ARTAB_REQUIRE(a.n_ctx > 0 && a.n_splits >= 1, ARTAB_EINVAL, "context attention: empty context or no splits");
  return a.dtype == ARTAB_BF16 ? launch_ctx_t<__nv_bfloat16>(a, s) : launch_ctx_t<float>(a, s);
}

int launch_buf_merge(const BufMergeArgs& a, cudaStream_t s) {
  if (a.n_items <= 0) return ARTAB_OK;
  if (a.mode_tf != 2 && buf_mma_supported(a.dtype, a.head_dim)) return launch_buf_merge_mma(a, s);
  return a.dtype == ARTAB_BF16 ? launch_buf_t<__nv_bfloat16>(a, s) : launch_buf_t<float>(a, s);
}

int launch_kv_append(int dtype, void* kv, const void* k_new, const void* v_new, long n_bh, int dh, int max_buf,
                     int pos, cudaStream_t s) {
  const long n = n_bh * dh;
  if (n <= 0) return ARTAB_OK;
  const unsigned grid = (unsigned)((n + 255) / 256);
  prof_begin(PROF_APPEND, s);
  if (dtype == ARTAB_BF16)
    kv_append_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)kv, (const __nv_bfloat16*)k_new,
                                                        (const __nv_bfloat16*)v_new, n_bh, dh, max_buf, pos);
  else
    kv_append_kernel<float><<<grid, 256, 0, s>>>((float*)kv, (const float*)k_new, (const float*)v_new, n_bh, dh,
                                                 max_buf, pos);
  prof_end(s);
  count_launch();
  return check_launch("kv_append_kernel");
}

}  // namespace artab
