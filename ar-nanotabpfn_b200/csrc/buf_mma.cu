// Private-buffer pass + log-sum-exp merge on warp-level tensor-core MMAs (bf16 caches, head_dim 32).
//
// Same job and the same one-warp-per-(stream, head[, item]) mapping as buf_merge_kernel, but the two
// queries of an item are rows 0 and 1 of an m16n8k16 A fragment, so a block of 16 keys costs
// 4 (Q.K^T) + 8 (P.V with P split into bf16 hi + lo, which keeps P at fp32 accuracy) MMAs and a
// two-value softmax per lane instead of ~140 scalar instructions.  A key's K row and V row are
// adjacent in memory, so a block of 16 keys is one contiguous 2 KB span: it goes through a 4-slot
// shared-memory ring filled with 16-byte cp.async copies and is read with ldmatrix (K^T fragments)
// and ldmatrix.trans (V fragments).
// At short buffers (a decode step of 512 streams) the pass is instruction-bound, at long ones it
// is a pure HBM stream; both get the shorter instruction stream.
#include "attn.cuh"

namespace artab {

namespace {

constexpr int DH = 32;     // head_dim served by this kernel
constexpr int KB = 16;     // keys per block (the k extent of one P.V MMA)
constexpr int NR = 4;      // V ring slots per warp
constexpr int PITCH = 144; // bytes per staged key: K row (64) + V row (64) + 16 of padding (conflict-free ldmatrix)
constexpr int WPB = 4;     // warps per CTA

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  // rows 8-15 of A (fragment registers a1, a3) are always zero here: only two query rows exist
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr)
               : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t saddr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr)
               : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t saddr, const void* gptr, bool valid) {
  const uint32_t n = valid ? 16u : 0u;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(saddr), "l"(gptr), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {  // MUFU ex2: exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(WPB * 32, 6) buf_mma_kernel(const BufMergeArgs a) {
  __shared__ __align__(16) uint8_t vs[WPB][NR][KB * PITCH];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // The dependent of this kernel is always a dense chain, which reads nothing but model constants
  // before its own wait: it may become resident (barriers, tensor-memory allocation, first weight
  // tiles) while this kernel is still walking the private buffers.  Its wait still covers everything
  // older, because this grid only completes after its own wait below.
  dep_trigger();
  if (threadIdx.x == 0) ARTAB_STAMP(3, 0);
  const long item = (long)blockIdx.x * WPB + warp;
  if (item >= a.n_items) return;  // warp-uniform; the kernel has no CTA-wide barrier
  const int g = lane >> 2;   // fragment row: query index (rows 0, 1) / key inside an 8-key tile
  const int t4 = lane & 3;   // fragment column pair

  long b;
  int h, len;
  long rows2[2];
  if (a.mode_tf) {
    const int ips = a.nt + 1;
    const int i = (int)(item % ips);
    const long bh = item / ips;
    b = bh / a.n_heads;
    h = (int)(bh - b * a.n_heads);
    len = i;
    rows2[0] = i < a.nt ? b * 2 * a.nt + a.nt + i : -1;
    rows2[1] = i >= 1 ? b * 2 * a.nt + i - 1 : -1;
  } else {
    b = item / a.n_heads;
    h = (int)(item - b * a.n_heads);
    len = a.lens ? min(max(__ldg(a.lens + b), 0), a.len0) : a.len0;
    rows2[0] = b * a.n_new + a.n_new - 1;
    rows2[1] = a.n_new == 2 ? b * a.n_new : -1;
  }

  // A fragments of Q for the two 16-wide k-steps: row g = query g, columns t4*2 + {0,1} (+8)
  uint32_t qa[2][2] = {{0u, 0u}, {0u, 0u}};
  if (g < 2 && rows2[g] >= 0) {
    const uint32_t* qp = reinterpret_cast<const uint32_t*>(reinterpret_cast<const __nv_bfloat16*>(a.q) +
                                                           ((size_t)rows2[g] * a.n_heads + h) * DH) + t4;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      qa[ks][0] = __ldg(qp + 8 * ks);
      qa[ks][1] = __ldg(qp + 8 * ks + 4);
    }
  }
  const __nv_bfloat16* kv =
      reinterpret_cast<const __nv_bfloat16*>(a.kv_buf) + ((size_t)(b * a.n_heads + h) * a.max_buf) * 2 * DH;
  const float sc = a.scale * kLog2e;
  const int nblk = (len + KB - 1) / KB;

  // K and V rows of block kb -> ring slot kb % NR: 16 keys x 8 chunks of 16 bytes (a key's K row and
  // V row are adjacent in memory), four chunks per lane, fully coalesced
  const uint32_t vs_base = smem_u32(&vs[warp][0][0]);
  auto stage = [&](int kb) {
    if (kb < nblk) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = i * 32 + lane, key = c >> 3, part = c & 7;
        const int gkey = kb * KB + key;
        const bool valid = gkey < len;
        const __nv_bfloat16* src = kv + (valid ? ((size_t)gkey * 2 * DH + part * 8) : 0);
        cp_async16(vs_base + (uint32_t)((kb % NR) * (KB * PITCH) + key * PITCH + part * 16), src, valid);
      }
    }
    cp_async_commit();  // one group per call, empty or not: the wait below counts groups
  };

  float m = -INFINITY, l = 0.f;
  float o[4][4];  // [8-dim tile][c0..c3]: c0, c1 = row g, dims tile*8 + t4*2 + {0,1}; c2, c3 stay zero
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;

#pragma unroll
  for (int i = 0; i < NR - 1; ++i) stage(i);
  const int mi = lane >> 3, r8 = lane & 7;  // ldmatrix: lane -> (matrix, row) whose address it supplies

  for (int kb = 0; kb < nblk; ++kb) {
    stage(kb + NR - 1);  // into the slot read in the previous iteration (its fragments were consumed)
    cp_async_wait<NR - 1>();  // block kb has landed once all but the NR - 1 newest groups are complete
    __syncwarp();
    const uint32_t slot = vs_base + (uint32_t)((kb % NR) * (KB * PITCH));

    // Scores of 16 keys for the two queries.  B fragments of K^T = plain ldmatrix of [8 keys][8 dims]
    // blocks; the four matrices of a call are dims 0-7, 8-15 (k-step 0) and 16-23, 24-31 (k-step 1).
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      uint32_t kf[4];
      ldmatrix_x4(slot + (uint32_t)((nt * 8 + r8) * PITCH + mi * 16), kf);
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
      mma_bf16(s[nt], qa[0][0], qa[0][1], kf[0], kf[1]);
      mma_bf16(s[nt], qa[1][0], qa[1][1], kf[2], kf[3]);
    }
    // this lane's four scores of row g: keys kb*16 + nt*8 + t4*2 + {0, 1}
    const int key0 = kb * KB + t4 * 2;
    float sv[4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) sv[nt * 2 + e] = key0 + nt * 8 + e < len ? s[nt][e] * sc : -INFINITY;
    float bm = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 2));   // finite: key kb*16 of every block is valid
    const float m_new = fmaxf(m, bm);
    const float alpha = fast_exp2(m - m_new);              // first block: exp2(-inf) = 0
    float p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = fast_exp2(sv[i] - m_new);
    l = l * alpha + (p[0] + p[1]) + (p[2] + p[3]);         // this lane's share of the row sum
    m = m_new;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[j][0] *= alpha;
      o[j][1] *= alpha;
    }
    // P as the A operand of P.V (k = 16 keys): a0 = keys t4*2+{0,1}, a2 = the same + 8; hi + lo parts
    const uint32_t ph0 = pack_bf16(p[0], p[1]), ph1 = pack_bf16(p[2], p[3]);
    const uint32_t pl0 = pack_bf16(p[0] - __uint_as_float(ph0 << 16), p[1] - __uint_as_float(ph0 & 0xffff0000u));
    const uint32_t pl1 = pack_bf16(p[2] - __uint_as_float(ph1 << 16), p[3] - __uint_as_float(ph1 & 0xffff0000u));
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      // V fragments (ldmatrix.trans of [8 keys][8 dims] blocks of the V half of the staged rows):
      // (dim tile 2c, keys 0-7), (2c, keys 8-15), (2c+1, keys 0-7), (2c+1, keys 8-15)
      uint32_t vb[4];
      ldmatrix_x4_trans(slot + (uint32_t)(((mi & 1) * 8 + r8) * PITCH + 64 + (2 * c + (mi >> 1)) * 16), vb);
      mma_bf16(o[2 * c], ph0, ph1, vb[0], vb[1]);
      mma_bf16(o[2 * c], pl0, pl1, vb[0], vb[1]);
      mma_bf16(o[2 * c + 1], ph0, ph1, vb[2], vb[3]);
      mma_bf16(o[2 * c + 1], pl0, pl1, vb[2], vb[3]);
    }
  }
  cp_async_wait<0>();
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);

  // The pass above read only what kernels older than the preceding one wrote (q and the buffer
  // rows); the context partials come from the preceding kernel.
  if (threadIdx.x == 0) ARTAB_STAMP(3, 3);
  dep_wait();
  if (threadIdx.x == 0) ARTAB_STAMP(3, 1);

  if (g >= 2 || rows2[g & 1] < 0) return;
  const long r = rows2[g];
  const float lse_b = l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;  // natural log, like the partials
  // Log-sum-exp merge with the context partials.  A dependent global load costs about a microsecond
  // here, so the partials are fetched four at a time with every load (LSEs and outputs) issued before
  // anything is computed, and folded in with a running reference `top` (rescaled when a chunk raises it).
  float top = lse_b, wsum = l > 0.f ? 1.0f : 0.f, out[8];
  {
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      out[2 * j] = o[j][0] * inv;
      out[2 * j + 1] = o[j][1] * inv;
    }
  }
  for (int sp0 = 0; sp0 < a.n_splits; sp0 += 4) {
    float ls[4];
    float2 ov[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int sp = min(sp0 + i, a.n_splits - 1);   // clamped: the loads never depend on a branch
      const size_t ro = ((size_t)sp * a.rows + r) * a.n_heads + h;
      ls[i] = __ldcg(a.lse_part + ro);
      const float* op = a.o_part + ro * DH + t4 * 2;
#pragma unroll
      for (int j = 0; j < 4; ++j) ov[i][j] = __ldcg(reinterpret_cast<const float2*>(op + 8 * j));
    }
    float cmax = -INFINITY;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (sp0 + i >= a.n_splits) ls[i] = -INFINITY;
      cmax = fmaxf(cmax, ls[i]);
    }
    if (cmax == -INFINITY) continue;
    const float ntop = fmaxf(top, cmax);
    const float rs = top == -INFINITY ? 0.f : expf(top - ntop);
    top = ntop;
    wsum *= rs;
#pragma unroll
    for (int j = 0; j < 8; ++j) out[j] *= rs;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float ws = ls[i] == -INFINITY ? 0.f : expf(ls[i] - top);
      wsum += ws;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        out[2 * j] = fmaf(ws, ov[i][j].x, out[2 * j]);
        out[2 * j + 1] = fmaf(ws, ov[i][j].y, out[2 * j + 1]);
      }
    }
  }
  if (a.lse_out && t4 == 0) a.lse_out[(size_t)r * a.n_heads + h] = wsum > 0.f ? top + logf(wsum) : -INFINITY;
  float inv = wsum > 0.f ? 1.0f / wsum : 0.f;
  if (a.poison_if && __ldcg(a.poison_if) != 0) inv = __int_as_float(0x7fc00000);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int col = h * DH + 8 * j + t4 * 2;
    float* dst = a.out + (a.out_lane_major ? lane_major_index(r, col, a.n_heads * DH) : (size_t)r * a.n_heads * DH + col);
    *reinterpret_cast<float2*>(dst) = make_float2(out[2 * j] * inv, out[2 * j + 1] * inv);
  }
  if (threadIdx.x == 0) ARTAB_STAMP(3, 2);
}


// ---------------------------------------------------------------------------------------------------
// Teacher forcing: item i of a stream is {target i, buffer token i - 1}, both seeing the stream's
// buffer keys [0, i).  One item per warp (the kernel above) reads the prefix of every item again and
// fills 2 of the 16 rows of every MMA.  Here a warp takes EIGHT consecutive items i0 .. i0 + 7 of one
// (stream, head): fragment row g is target i0 + g, row g + 8 is buffer token i0 + g - 1, so a lane's
// two rows belong to the same item and share its visible length i0 + g.  The warp walks the keys
// [0, i0 + 7) once: an eighth of the key traffic and of the MMAs, at twice the softmax work per block.
// A row with no visible key so far (the rows of item 0 never have one) keeps its maximum at -inf; the
// exponent reference is then replaced by 0, so that exp2(-inf - 0) = 0 and nothing turns into NaN.
// ---------------------------------------------------------------------------------------------------
constexpr int TFG = 8;  // items per warp

__device__ __forceinline__ void mma_bf16_full(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(WPB * 32, 5) buf_mma_tf_kernel(const BufMergeArgs a, const long n_groups) {
  __shared__ __align__(16) uint8_t vs[WPB][NR][KB * PITCH];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  dep_trigger();  // see buf_mma_kernel: the dependent dense chain reads only model constants before its wait
  const long grp = (long)blockIdx.x * WPB + warp;
  if (grp >= n_groups) return;  // warp-uniform; the kernel has no CTA-wide barrier
  const int g = lane >> 2, t4 = lane & 3;
  const int gps = (a.nt + 1 + TFG - 1) / TFG;   // groups per (stream, head)
  const int i0 = (int)(grp % gps) * TFG;
  const long bh = grp / gps;
  const long b = bh / a.n_heads;
  const int h = (int)(bh - b * a.n_heads);
  const int item = i0 + g;                      // this lane's item: rows g (target) and g + 8 (buffer token)
  const int len_row = min(item, a.nt);          // keys [0, len_row) are visible to both of its rows
  const long row_t = item < a.nt ? b * 2 * a.nt + a.nt + item : -1;
  const long row_b = (item >= 1 && item <= a.nt) ? b * 2 * a.nt + item - 1 : -1;
  const int len = min(i0 + TFG - 1, a.nt);      // keys the warp walks

  // A fragments of Q for the two 16-wide k-steps: a0 / a2 = row g, a1 / a3 = row g + 8
  uint32_t qt[2][2] = {{0u, 0u}, {0u, 0u}}, qb[2][2] = {{0u, 0u}, {0u, 0u}};
  const __nv_bfloat16* qbase = reinterpret_cast<const __nv_bfloat16*>(a.q);
  if (row_t >= 0) {
    const uint32_t* qp = reinterpret_cast<const uint32_t*>(qbase + ((size_t)row_t * a.n_heads + h) * DH) + t4;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      qt[ks][0] = __ldg(qp + 8 * ks);
      qt[ks][1] = __ldg(qp + 8 * ks + 4);
    }
  }
  if (row_b >= 0) {
    const uint32_t* qp = reinterpret_cast<const uint32_t*>(qbase + ((size_t)row_b * a.n_heads + h) * DH) + t4;
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
      qb[ks][0] = __ldg(qp + 8 * ks);
      qb[ks][1] = __ldg(qp + 8 * ks + 4);
    }
  }
  const __nv_bfloat16* kv =
      reinterpret_cast<const __nv_bfloat16*>(a.kv_buf) + ((size_t)(b * a.n_heads + h) * a.max_buf) * 2 * DH;
  const float sc = a.scale * kLog2e;
  const int nblk = (len + KB - 1) / KB;
  const uint32_t vs_base = smem_u32(&vs[warp][0][0]);
  auto stage = [&](int kb) {
    if (kb < nblk) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = i * 32 + lane, key = c >> 3, part = c & 7;
        const int gkey = kb * KB + key;
        const bool valid = gkey < len;
        const __nv_bfloat16* src = kv + (valid ? ((size_t)gkey * 2 * DH + part * 8) : 0);
        cp_async16(vs_base + (uint32_t)((kb % NR) * (KB * PITCH) + key * PITCH + part * 16), src, valid);
      }
    }
    cp_async_commit();
  };

  float mt = -INFINITY, mb = -INFINITY, lt = 0.f, lb = 0.f;   // running maximum and row sum of the two rows
  float o[4][4];  // [8-dim tile]: c0, c1 = row g (target), c2, c3 = row g + 8 (buffer token)
#pragma unroll
  for (int j = 0; j < 4; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[j][e] = 0.f;
#pragma unroll
  for (int i = 0; i < NR - 1; ++i) stage(i);
  const int mi = lane >> 3, r8 = lane & 7;

  for (int kb = 0; kb < nblk; ++kb) {
    stage(kb + NR - 1);
    cp_async_wait<NR - 1>();
    __syncwarp();
    const uint32_t slot = vs_base + (uint32_t)((kb % NR) * (KB * PITCH));
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      uint32_t kf[4];
      ldmatrix_x4(slot + (uint32_t)((nt * 8 + r8) * PITCH + mi * 16), kf);
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
      mma_bf16_full(s[nt], qt[0][0], qb[0][0], qt[0][1], qb[0][1], kf[0], kf[1]);
      mma_bf16_full(s[nt], qt[1][0], qb[1][0], qt[1][1], qb[1][1], kf[2], kf[3]);
    }
    // this lane's scores: keys kb*16 + nt*8 + t4*2 + {0, 1}; [nt][0..1] row g, [nt][2..3] row g + 8
    const int key0 = kb * KB + t4 * 2;
    float st[4], sb[4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const bool vis = key0 + nt * 8 + e < len_row;
        st[nt * 2 + e] = vis ? s[nt][e] * sc : -INFINITY;
        sb[nt * 2 + e] = vis ? s[nt][2 + e] * sc : -INFINITY;
      }
    float bt = fmaxf(fmaxf(st[0], st[1]), fmaxf(st[2], st[3]));
    float bb = fmaxf(fmaxf(sb[0], sb[1]), fmaxf(sb[2], sb[3]));
    bt = fmaxf(bt, __shfl_xor_sync(0xffffffffu, bt, 1));
    bt = fmaxf(bt, __shfl_xor_sync(0xffffffffu, bt, 2));
    bb = fmaxf(bb, __shfl_xor_sync(0xffffffffu, bb, 1));
    bb = fmaxf(bb, __shfl_xor_sync(0xffffffffu, bb, 2));
    const float mt_new = fmaxf(mt, bt), mb_new = fmaxf(mb, bb);
    const float mt_use = mt_new == -INFINITY ? 0.f : mt_new;   // nothing visible yet: exp2(-inf - 0) = 0
    const float mb_use = mb_new == -INFINITY ? 0.f : mb_new;
    const float at = fast_exp2(mt - mt_use), ab = fast_exp2(mb - mb_use);   // old maximum -inf: 0, like the sums
    float pt[4], pb[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      pt[i] = fast_exp2(st[i] - mt_use);
      pb[i] = fast_exp2(sb[i] - mb_use);
    }
    lt = lt * at + (pt[0] + pt[1]) + (pt[2] + pt[3]);
    lb = lb * ab + (pb[0] + pb[1]) + (pb[2] + pb[3]);
    mt = mt_new;
    mb = mb_new;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[j][0] *= at;
      o[j][1] *= at;
      o[j][2] *= ab;
      o[j][3] *= ab;
    }
    // P as the A operand of P.V (k = 16 keys), hi + lo parts: a0 / a2 row g, a1 / a3 row g + 8
    const uint32_t th0 = pack_bf16(pt[0], pt[1]), th1 = pack_bf16(pt[2], pt[3]);
    const uint32_t bh0 = pack_bf16(pb[0], pb[1]), bh1 = pack_bf16(pb[2], pb[3]);
    const uint32_t tl0 = pack_bf16(pt[0] - __uint_as_float(th0 << 16), pt[1] - __uint_as_float(th0 & 0xffff0000u));
    const uint32_t tl1 = pack_bf16(pt[2] - __uint_as_float(th1 << 16), pt[3] - __uint_as_float(th1 & 0xffff0000u));
    const uint32_t bl0 = pack_bf16(pb[0] - __uint_as_float(bh0 << 16), pb[1] - __uint_as_float(bh0 & 0xffff0000u));
    const uint32_t bl1 = pack_bf16(pb[2] - __uint_as_float(bh1 << 16), pb[3] - __uint_as_float(bh1 & 0xffff0000u));
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t vb[4];
      ldmatrix_x4_trans(slot + (uint32_t)(((mi & 1) * 8 + r8) * PITCH + 64 + (2 * c + (mi >> 1)) * 16), vb);
      mma_bf16_full(o[2 * c], th0, bh0, th1, bh1, vb[0], vb[1]);
      mma_bf16_full(o[2 * c], tl0, bl0, tl1, bl1, vb[0], vb[1]);
      mma_bf16_full(o[2 * c + 1], th0, bh0, th1, bh1, vb[2], vb[3]);
      mma_bf16_full(o[2 * c + 1], tl0, bl0, tl1, bl1, vb[2], vb[3]);
    }
  }
  cp_async_wait<0>();
  lt += __shfl_xor_sync(0xffffffffu, lt, 1);
  lt += __shfl_xor_sync(0xffffffffu, lt, 2);
  lb += __shfl_xor_sync(0xffffffffu, lb, 1);
  lb += __shfl_xor_sync(0xffffffffu, lb, 2);

  // The pass above read only what kernels older than the preceding one wrote (q and the buffer
  // rows); the context partials come from the preceding kernel.
  dep_wait();

#pragma unroll
  for (int w = 0; w < 2; ++w) {   // w = 0: the target row (c0, c1), w = 1: the buffer-token row (c2, c3)
    const long r = w ? row_b : row_t;
    if (r < 0) continue;
    const float l = w ? lb : lt, m = w ? mb : mt;
    const float lse_b = l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;  // natural log, like the partials
    float top = lse_b, wsum = l > 0.f ? 1.0f : 0.f, out[8];
    {
      const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        out[2 * j] = o[j][2 * w] * inv;
        out[2 * j + 1] = o[j][2 * w + 1] * inv;
      }
    }
    for (int sp0 = 0; sp0 < a.n_splits; sp0 += 4) {
      float ls[4];
      float2 ov[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int sp = min(sp0 + i, a.n_splits - 1);
        const size_t ro = ((size_t)sp * a.rows + r) * a.n_heads + h;
        ls[i] = __ldcg(a.lse_part + ro);
        const float* op = a.o_part + ro * DH + t4 * 2;
#pragma unroll
        for (int j = 0; j < 4; ++j) ov[i][j] = __ldcg(reinterpret_cast<const float2*>(op + 8 * j));
      }
      float cmax = -INFINITY;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (sp0 + i >= a.n_splits) ls[i] = -INFINITY;
        cmax = fmaxf(cmax, ls[i]);
      }
      if (cmax == -INFINITY) continue;
      const float ntop = fmaxf(top, cmax);
      const float rs = top == -INFINITY ? 0.f : expf(top - ntop);
      top = ntop;
      wsum *= rs;
#pragma unroll
      for (int j = 0; j < 8; ++j) out[j] *= rs;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float ws = ls[i] == -INFINITY ? 0.f : expf(ls[i] - top);
        wsum += ws;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          out[2 * j] = fmaf(ws, ov[i][j].x, out[2 * j]);
          out[2 * j + 1] = fmaf(ws, ov[i][j].y, out[2 * j + 1]);
        }
      }
    }
    if (a.lse_out && t4 == 0) a.lse_out[(size_t)r * a.n_heads + h] = wsum > 0.f ? top + logf(wsum) : -INFINITY;
    float inv = wsum > 0.f ? 1.0f / wsum : 0.f;
    if (a.poison_if && __ldcg(a.poison_if) != 0) inv = __int_as_float(0x7fc00000);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = h * DH + 8 * j + t4 * 2;
      float* dst = a.out + (a.out_lane_major ? lane_major_index(r, col, a.n_heads * DH) : (size_t)r * a.n_heads * DH + col);
      *reinterpret_cast<float2*>(dst) = make_float2(out[2 * j] * inv, out[2 * j + 1] * inv);
    }
  }
}

}  // namespace

bool buf_mma_supported(int dtype, int head_dim) { return dtype == ARTAB_BF16 && head_dim == DH; }

int launch_buf_merge_mma(const BufMergeArgs& a, cudaStream_t s) {
  if (a.n_items <= 0) return ARTAB_OK;
  ARTAB_REQUIRE(buf_mma_supported(a.dtype, a.head_dim), ARTAB_EINVAL, "buffer attention (mma): bf16, head_dim 32 only");
  prof_begin(PROF_BUF, s);
  ARTAB_STAMP_ATTACH();
  cudaError_t le;
  if (a.mode_tf == 1) {   // teacher forcing: eight items of a (stream, head) per warp
    const long per_stream_head = a.nt + 1;
    const long n_groups = a.n_items / per_stream_head * ((per_stream_head + TFG - 1) / TFG);
    const unsigned grid = (unsigned)((n_groups + WPB - 1) / WPB);
    le = launch_dependent(buf_mma_tf_kernel, dim3(grid), dim3(WPB * 32), 0, s, a, n_groups);
  } else {
    const unsigned grid = (unsigned)((a.n_items + WPB - 1) / WPB);
    le = launch_dependent(buf_mma_kernel, dim3(grid), dim3(WPB * 32), 0, s, a);
  }
  prof_end(s);
  ARTAB_REQUIRE(le == cudaSuccess, ARTAB_ELAUNCH, "buf_mma_kernel: %s", cudaGetErrorString(le));
  count_launch();
  return check_launch("buf_mma_kernel");
}

}  // namespace artab
