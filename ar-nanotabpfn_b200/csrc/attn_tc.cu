// Shared-context attention on the 5th-generation tensor cores (sm_100a).
//
// Queries of every sample stream are stacked into 128-row M tiles and contracted
// against the shared context K/V: S = Q.K^T and O = P.V are tcgen05.mma
// instructions with the accumulators in tensor memory (TMEM); Q, K and V^T tiles
// arrive in shared memory by TMA (plain per-CTA loads) in the
// swizzled K-major layouts the MMA descriptors name.  Softmax runs on two warpgroups
// that split a key tile's 128 score columns and own one query row per thread
// (TMEM lane == row); the running max / sum / output stay in registers and P goes
// back to the tensor core through its own TMEM columns as packed bf16.  V is kept as
// a bf16 hi part and a bf16 lo part, so O = P.[V_hi | V_lo] has 64 columns.
//
// One CTA = one (M tile, head, context group, key split).  Warp 0 issues TMA,
// warp 1 issues MMA and owns the TMEM allocation, warps 2-5 and 6-9 do softmax.
// The next tile's Q.K^T is issued as soon as every softmax thread has its scores in
// registers, so it overlaps the exponentials; P has one buffer, so it is rewritten only
// once the previous P.V has completed.  Two CTAs are resident per SM (256 TMEM
// columns each), so the MMA of one overlaps the softmax of the other.  Every mbarrier
// wait is bounded: on expiry the CTA raises its abort flag, records a code in the
// status word, drains its own copies, frees its TMEM and returns.
//
// Output per (split, row, head): normalised O [32] fp32 and the natural-log LSE,
// merged later with the private-buffer pass (buf_mma_kernel / buf_merge_kernel).
#include <cuda.h>

#include "attn.cuh"

namespace artab {

namespace {

constexpr int BM = 128;       // query rows per tile
constexpr int BN = 128;       // keys per tile
constexpr int DH = 32;        // head dim this kernel is built for
constexpr int NSTAGE = 3;     // K/V pipeline depth
constexpr int kThreads = 320; // warp 0 TMA, warp 1 MMA, warps 2-5 and 6-9 softmax (two warpgroups)
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0;    // S: 128 fp32 columns
constexpr uint32_t kColO = 128;  // O tile: 64 fp32 columns = P.V_hi | P.V_lo
constexpr uint32_t kColP = 192;  // P: 128 bf16 = 64 packed columns (A operand of P.V)
constexpr long long kWaitCycles = 2000000000LL;  // about one second

// Abort flag of the CTA and, right behind it, the limit of every bounded wait in SM clock cycles (a
// launch parameter): a wait site hands over the flag's address and finds the limit next to it.
struct WaitCtl {
  int abort_flag;
  int pad;
  long long limit;
};

struct __align__(1024) Smem {
  uint8_t q[BM * 64];               // [128 rows][32 bf16], 64-byte swizzle
  uint8_t k[NSTAGE][BN * 64];       // [128 keys][32 bf16], 64-byte swizzle
  uint8_t v[NSTAGE][2][64 * 128];   // V^T hi|lo: two boxes of [64 rows][64 keys], 128-byte swizzle
  uint64_t q_full, s_full, p_full, o_full;
  uint64_t s_free;                  // every softmax thread has read its scores of the current tile
  uint64_t kv_full[NSTAGE], kv_empty[NSTAGE];
  float xmax[2][2][BM];             // row maxima exchanged between the two softmax warpgroups
  float xsum[BM];                   // row sum of the second warpgroup (epilogue)
  uint32_t tmem_base;
  uint32_t pad_;
  WaitCtl ctl;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
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
// Bounded wait: false when the CTA is aborting (this wait or another one gave up).
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(b, parity)) return true;
  const long long limit = reinterpret_cast<volatile WaitCtl*>(abort_flag)->limit;
  const long long t0 = clock64();
  for (;;) {
    if (mbar_try(b, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > limit) {
      *abort_flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tm, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(tm), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// K-major shared-memory matrix descriptor: rows of `swizzle` bytes, 8-row groups `sbo` bytes apart.
constexpr uint64_t kLayoutSw128 = 2, kLayoutSw64 = 4;
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t sbo_bytes, uint64_t layout) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;                  // leading byte offset: unused for swizzled K-major
  d |= (uint64_t)(sbo_bytes >> 4) << 32;   // stride byte offset
  d |= (uint64_t)1 << 46;                  // descriptor version (sm_100)
  d |= layout << 61;
  return d;
}

// kind::f16 instruction descriptor: fp32 accumulate, bf16 A and B, both K-major.
constexpr uint32_t make_idesc(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for two values on the FMA pipe instead of the special-function unit (which delivers only 16
// exponentials per clock and SM and is what bounds this kernel at head_dim 32): round x to the nearest
// integer n with the 1.5 * 2^23 trick, a cubic for 2^f on f = x - n in [-0.5, 0.5] (relative error
// 7.5e-5, far below the bf16 rounding of P), and n added into the exponent field.  x is clamped at
// -125 (the result is then ~2e-38, i.e. nothing); x stays below ~2^4 here (lazy maximum).
#ifndef ARTAB_POLY_EXP_OF_8
#define ARTAB_POLY_EXP_OF_8 2   // of every 8 score pairs this many take the FMA-pipe exponential (measured best: 0 -> 88.2 us, 2 -> 82.2, 3 -> 85.3, 4 -> 89.7 at 4096 rows x 8192 keys)
#endif
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  x.x = fmaxf(x.x, -125.0f);
  x.y = fmaxf(x.y, -125.0f);
  float2 xf, p;
  asm("{\n\t.reg .b64 rx, rm, rn, rf, rr, rp, c3, c2, c1, c0, m1;\n\t"
      "mov.b64 rx, {%4, %5};\n\t"
      "mov.b64 rm, {%6, %6};\n\t"
      "mov.b64 rn, {%7, %7};\n\t"
      "mov.b64 m1, {%8, %8};\n\t"
      "mov.b64 c3, {%9, %9};\n\t"
      "mov.b64 c2, {%10, %10};\n\t"
      "mov.b64 c1, {%11, %11};\n\t"
      "mov.b64 c0, {%12, %12};\n\t"
      "add.rn.f32x2 rf, rx, rm;\n\t"          // x + 1.5 * 2^23: the integer lands in the low mantissa bits
      "add.rn.f32x2 rr, rf, rn;\n\t"          // round(x)
      "fma.rn.f32x2 rr, rr, m1, rx;\n\t"      // f = x - round(x)
      "fma.rn.f32x2 rp, c3, rr, c2;\n\t"
      "fma.rn.f32x2 rp, rp, rr, c1;\n\t"
      "fma.rn.f32x2 rp, rp, rr, c0;\n\t"
      "mov.b64 {%0, %1}, rf;\n\t"
      "mov.b64 {%2, %3}, rp;\n\t}"
      : "=f"(xf.x), "=f"(xf.y), "=f"(p.x), "=f"(p.y)
      : "f"(x.x), "f"(x.y), "f"(12582912.0f), "f"(-12582912.0f), "f"(-1.0f), "f"(0.0551716685f), "f"(0.2426111251f),
        "f"(0.6932609677f), "f"(0.9999280572f));
  return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(xf.x) << 23)),
                     __int_as_float(__float_as_int(p.y) + (__float_as_int(xf.y) << 23)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct TcParams {
  int rows, rows_per_group, n_groups, n_heads, n_ctx, n_ctx_pad, n_splits;
  float scale_log2e;
  int out_lane_major;
  int kv_stable;  // the context K/V were written long before the preceding kernel: prefetch them early
  float* out;
  float* lse;
  int32_t* status;
  long long wait_cycles;  // limit of every mbarrier wait, in SM clock cycles
  int drop_score_commits; // diagnostics only: the MMA thread never signals "scores ready", so the waits run out
};

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]),
        "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

// How far (in log2 units) a row's running reference may lag behind its true maximum before the
// accumulated output is rescaled: exponentials then stay below 2^8, far inside bf16 / fp32 range.
constexpr float kLazyMax = 8.0f;

// Softmax of this thread's half (64 columns) of one 128 x 128 score tile row.  The two
// softmax warpgroups own columns [0,64) and [64,128) of the same rows and exchange their row
// maxima through shared memory.  MASKED: columns >= n_valid are -inf.
//
// O accumulates in tensor memory across the key tiles (the P.V MMAs run with the accumulate flag), so
// no thread folds it tile by tile.  The exponentials are taken against a reference m that is only
// raised when a tile's maximum exceeds it by more than kLazyMax; then O is rescaled in place (each
// warpgroup its half of the 64 output columns: one tcgen05.ld / st round trip), which on ordinary
// data happens on the first tiles only.  The result does not depend on when m is raised: the final
// O / l and lse = m + log2(l) are exact in m.
template <bool MASKED>
__device__ __forceinline__ bool softmax_tile(Smem* sm, uint32_t t_row, int wg, int row, int parity, float sc,
                                             int n_valid, float& m, float& l, bool first,
                                             volatile int* abort_flag) {
  uint32_t r[32];
  float mx = -INFINITY;
  const int col0 = 64 * wg;
#pragma unroll 1  // one 32-column chunk in flight keeps the register count low enough for two CTAs per SM
  for (int c = 0; c < 2; ++c) {
    tmem_ld32(t_row + kColS + col0 + 32 * c, r);
    tmem_wait_ld();
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      float s = __uint_as_float(r[i]);
      if (MASKED && col0 + 32 * c + i >= n_valid) s = -INFINITY;
      mx = fmaxf(mx, s);
    }
  }
  sm->xmax[parity][wg][row] = mx;
  asm volatile("bar.sync 2, 256;" ::: "memory");  // the two softmax warpgroups only
  mx = fmaxf(mx, sm->xmax[parity][wg ^ 1][row]) * sc;  // column 0 of every tile is valid, so mx is finite
  // both warpgroups see the same mx for the row and take the same decision
  const bool raise = first || mx > m + kLazyMax;
  const float alpha = raise ? ex2_approx(m - mx) : 1.0f;   // m = -inf on the first tile gives 0
  if (raise) m = mx;
  bool ok = true;
  float sum = 0.f;
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    tmem_ld32(t_row + kColS + col0 + 32 * c, r);
    tmem_wait_ld();
    if (c == 1) {  // the scores are in registers: the next tile's Q.K^T may overwrite them
      tc_fence_before();
      mbar_arrive(&sm->s_free);
    }
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float p0, p1;
      if (((i >> 1) & 7) < ARTAB_POLY_EXP_OF_8) {   // compile-time choice per unrolled pair
        const float2 e = ex2_poly2(make_float2(fmaf(__uint_as_float(r[i]), sc, -m), fmaf(__uint_as_float(r[i + 1]), sc, -m)));
        p0 = e.x;
        p1 = e.y;
      } else {
        p0 = ex2_approx(fmaf(__uint_as_float(r[i]), sc, -m));
        p1 = ex2_approx(fmaf(__uint_as_float(r[i + 1]), sc, -m));
      }
      if (MASKED) {
        if (col0 + 32 * c + i >= n_valid) p0 = 0.f;
        if (col0 + 32 * c + i + 1 >= n_valid) p1 = 0.f;
      }
      sum += p0 + p1;
      pk[i >> 1] = pack_bf16(p0, p1);
    }
    // This tile's scores were computed while the previous tile's P . V may still be running: P has
    // one buffer and O one accumulator, so both are touched only once that MMA has completed (the
    // maxima and the first half of the exponentials above overlapped it).
    if (c == 0 && !first) {
      ok = mbar_wait(&sm->o_full, parity ^ 1, abort_flag);
      tc_fence_after();
      if (__any_sync(0xffffffffu, raise)) {  // rare: rescale this warpgroup's half of the accumulated O
        uint32_t o[32];
        tmem_ld32(t_row + kColO + 32 * wg, o);
        tmem_wait_ld();
#pragma unroll
        for (int d = 0; d < 32; ++d) o[d] = __float_as_uint(__uint_as_float(o[d]) * alpha);
        tmem_st32(t_row + kColO + 32 * wg, o);
      }
    }
    tmem_st16(t_row + kColP + 32 * wg + 16 * c, pk);
  }
  l = l * alpha + sum;
  return ok;
}

__global__ void __launch_bounds__(kThreads, 2)
ctx_attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  Smem* sm = reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int g = blockIdx.z / p.n_splits, split = blockIdx.z - g * p.n_splits;
  const int rows_in_group = p.n_groups == 1 ? p.rows : p.rows_per_group;
  const long group_row0 = p.n_groups == 1 ? 0 : (long)g * p.rows_per_group;
  const int m0 = blockIdx.x * BM;
  if (threadIdx.x == 0) ARTAB_STAMP(2, 0);

  const int tiles = (p.n_ctx + BN - 1) / BN;
  const int tps = (tiles + p.n_splits - 1) / p.n_splits;
  const int tile_begin = split * tps;
  const int tile_end = min(tiles, tile_begin + tps);
  const int nt = tile_end - tile_begin;

  // softmax threads: TMEM lane (= tile row) owned by this thread; warpgroup 0 = warps 2-5, 1 = warps 6-9
  const int lane_base = 32 * (warp & 3);
  const int row = lane_base + lane;
  const int wg = warp >= 6 ? 1 : 0;
  const bool row_valid = warp >= 2 && warp < 6 && (m0 + row) < rows_in_group;  // warpgroup 0 stores
  const size_t out_row = ((size_t)split * p.rows + group_row0 + m0 + row) * p.n_heads + h;

  if (nt <= 0) {  // empty split: contributes nothing to the merge
    dep_wait();
    dep_trigger();
    if (row_valid) {
      float4* o = reinterpret_cast<float4*>(p.out + out_row * DH);
#pragma unroll
      for (int i = 0; i < DH / 4; ++i) o[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      p.lse[out_row] = -INFINITY;
    }
    return;
  }

  if (threadIdx.x == 0) {
    mbar_init(&sm->q_full, 1);
    mbar_init(&sm->s_full, 1);
    mbar_init(&sm->p_full, 256);
    mbar_init(&sm->o_full, 1);
    mbar_init(&sm->s_free, 256);
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&sm->kv_full[s], 1);
      mbar_init(&sm->kv_empty[s], 1);
    }
    sm->ctl.abort_flag = 0;
    sm->ctl.limit = p.wait_cycles;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm->tmem_base)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm->tmem_base;
  volatile int* abort_flag = &sm->ctl.abort_flag;
  if (warp != 0) {  // the producer waits after its early K/V prefetch
    dep_wait();
    dep_trigger();
    if (threadIdx.x == 32) ARTAB_STAMP(2, 1);
  }

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      const int krow0 = (g * p.n_heads + h) * p.n_ctx_pad;
      const int vrow0 = (g * p.n_heads + h) * 2 * DH;
      auto load_kv = [&](int j) {
        const int st = j % NSTAGE;
        const int key0 = (tile_begin + j) * BN;
        mbar_expect_tx(&sm->kv_full[st], BN * 64 + 2 * 64 * 128);
        tma_load_2d(sm->k[st], &tm_k, 0, krow0 + key0, &sm->kv_full[st]);
        tma_load_2d(sm->v[st][0], &tm_v, key0, vrow0, &sm->kv_full[st]);
        tma_load_2d(sm->v[st][1], &tm_v, key0 + 64, vrow0, &sm->kv_full[st]);
      };
      // the first ring of K/V tiles may be fetched while the preceding kernel (which produces Q) runs
      int issued = 0;
      const int early = p.kv_stable ? min(nt, NSTAGE) : 0;
      for (; issued < early; ++issued) load_kv(issued);
      dep_wait();
      mbar_expect_tx(&sm->q_full, BM * 64);
      tma_load_2d(sm->q, &tm_q, h * DH, (int)(group_row0 + m0), &sm->q_full);
      for (int j = issued; j < nt; ++j) {
        if (j >= NSTAGE && !mbar_wait(&sm->kv_empty[j % NSTAGE], ((j / NSTAGE) + 1) & 1, abort_flag)) break;
        load_kv(j);
        issued = j + 1;
      }
      if (*abort_flag) {  // drain our own copies before the CTA may exit
        {
          const long long t0 = clock64();
          while (!mbar_try(&sm->q_full, 0) && clock64() - t0 < p.wait_cycles) {
          }
        }
        for (int j = max(0, issued - NSTAGE); j < issued; ++j) {
          const long long t0 = clock64();
          while (!mbar_try(&sm->kv_full[j % NSTAGE], (j / NSTAGE) & 1) && clock64() - t0 < p.wait_cycles) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(BM, BN);
      constexpr uint32_t idesc_pv = make_idesc(BM, 2 * DH);
      bool ok = mbar_wait(&sm->q_full, 0, abort_flag);
      const uint32_t q_addr = smem_u32(sm->q);
      // S = Q . K^T of tile j   (M 128, N 128, K 32 = two k-steps of 16 bf16 = 32 bytes)
      auto issue_qk = [&](int j) -> bool {
        const int st = j % NSTAGE;
        if (!mbar_wait(&sm->kv_full[st], (j / NSTAGE) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sm->k[st]);
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
          umma_ss(tmem + kColS, make_desc(q_addr + 32 * ks, 512, kLayoutSw64),
                  make_desc(k_addr + 32 * ks, 512, kLayoutSw64), idesc_qk, ks);
        if (!p.drop_score_commits) umma_commit(&sm->s_full);
        return true;
      };
      ok = ok && issue_qk(0);
      for (int j = 0; ok && j < nt; ++j) {
        const int st = j % NSTAGE;
        // The next tile's scores are computed while the softmax threads still turn this tile's
        // into P: they release S as soon as their last score is in registers.
        if (j + 1 < nt) {
          ok = mbar_wait(&sm->s_free, j & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          ok = issue_qk(j + 1);
          if (!ok) break;
        }
        // softmax writes P (and has folded the previous O tile) -> O = P . [V_hi | V_lo]
        ok = mbar_wait(&sm->p_full, j & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t v_addr = smem_u32(sm->v[st][ks >> 2]) + 32 * (ks & 3);
          umma_ts(tmem + kColO, tmem + kColP + 8 * ks, make_desc(v_addr, 1024, kLayoutSw128), idesc_pv, (j | ks) != 0);
        }
        umma_commit(&sm->o_full);
        umma_commit(&sm->kv_empty[st]);
      }
    }
  } else {
    // --------------------------------- softmax ---------------------------------
    const uint32_t t_row = tmem + ((uint32_t)lane_base << 16);
    const float sc = p.scale_log2e;
    float m = -INFINITY, l = 0.f;
    uint32_t r[32];
    bool ok = true;
    // On an abort the loop still runs every iteration (waits return at once, results are void):
    // both warpgroups must execute the same number of bar.sync instructions.
    for (int j = 0; j < nt; ++j) {
      ok = mbar_wait(&sm->s_full, j & 1, abort_flag) && ok;
      tc_fence_after();
      const int n_valid = p.n_ctx - (tile_begin + j) * BN;
      if (n_valid >= BN)
        ok = softmax_tile<false>(sm, t_row, wg, row, j & 1, sc, BN, m, l, j == 0, abort_flag) && ok;
      else
        ok = softmax_tile<true>(sm, t_row, wg, row, j & 1, sc, n_valid, m, l, j == 0, abort_flag) && ok;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&sm->p_full);
    }
    if (wg == 1) sm->xsum[row] = l;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (wg == 0) {
      l += sm->xsum[row];
      if (ok) ok = mbar_wait(&sm->o_full, (nt - 1) & 1, abort_flag);
      if (ok) {
        tc_fence_after();
        float o[DH];
        tmem_ld32(t_row + kColO, r);          // P . V_hi
        tmem_wait_ld();
#pragma unroll
        for (int d = 0; d < DH; ++d) o[d] = __uint_as_float(r[d]);
        tmem_ld32(t_row + kColO + 32, r);     // P . V_lo
        tmem_wait_ld();
#pragma unroll
        for (int d = 0; d < DH; ++d) o[d] += __uint_as_float(r[d]);
        if (row_valid) {
          const float inv = 1.0f / l;
#pragma unroll
          for (int d = 0; d < DH; d += 4) {
            float* dst = p.out + (p.out_lane_major ? lane_major_index(group_row0 + m0 + row, h * DH + d, p.n_heads * DH)
                                                   : out_row * DH + d);
            *reinterpret_cast<float4*>(dst) = make_float4(o[d] * inv, o[d + 1] * inv, o[d + 2] * inv, o[d + 3] * inv);
          }
          p.lse[out_row] = (m + log2f(l)) * kLn2;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
  if (threadIdx.x == 0 && sm->ctl.abort_flag && p.status) atomicExch(p.status, 1);
  if (threadIdx.x == 0) ARTAB_STAMP(2, 2);
}

// ---------------------------------- host side ----------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// A tensor map depends only on (base, extents, pitch, box, swizzle): the decode loop asks for the same
// few maps hundreds of times per call (q once per row count, K and V once per layer), so the encoded
// descriptors are kept in a small per-thread table, replaced round-robin.
struct MapKey {
  const void* base;
  uint64_t inner, outer, row_bytes;
  uint32_t box_inner, box_outer;
  int swz;
  bool operator==(const MapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && row_bytes == o.row_bytes &&
           box_inner == o.box_inner && box_outer == o.box_outer && swz == o.swz;
  }
};
constexpr int kMapCache = 64;
struct MapCache {
  MapKey key[kMapCache];
  CUtensorMap map[kMapCache];
  int used = 0, next = 0;
};

int make_map_2d(CUtensorMap* tm, const void* base, uint64_t inner, uint64_t outer, uint64_t row_bytes, uint32_t box_inner,
                uint32_t box_outer, CUtensorMapSwizzle swz, const char* what) {
  static thread_local MapCache cache;
  const MapKey k{base, inner, outer, row_bytes, box_inner, box_outer, (int)swz};
  for (int i = 0; i < cache.used; ++i)
    if (cache.key[i] == k) {
      *tm = cache.map[i];
      return ARTAB_OK;
    }
  EncodeTiledFn fn = encode_fn();
  ARTAB_REQUIRE(fn, ARTAB_EDRIVER, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  ARTAB_REQUIRE(r == CUDA_SUCCESS, ARTAB_EINVAL, "tensor map for %s refused (CUresult %d): base %p, dims %llu x %llu",
                what, (int)r, base, (unsigned long long)inner, (unsigned long long)outer);
  const int slot = cache.used < kMapCache ? cache.used++ : (cache.next = (cache.next + 1) % kMapCache);
  cache.key[slot] = k;
  cache.map[slot] = *tm;
  return ARTAB_OK;
}

}  // namespace

bool ctx_attn_tc_supported(int dtype, int head_dim) { return dtype == ARTAB_BF16 && head_dim == DH; }

int launch_ctx_attn_tc(const CtxAttnArgs& a, cudaStream_t s) {
  if (a.rows <= 0) return ARTAB_OK;
  ARTAB_REQUIRE(a.dtype == ARTAB_BF16 && a.head_dim == DH && a.v_transposed, ARTAB_EINVAL,
                "tensor-core context attention needs bf16, head_dim 32 and a transposed V cache");
  ARTAB_REQUIRE(a.n_ctx > 0 && a.n_ctx_pad % 8 == 0 && a.n_splits >= 1, ARTAB_EINVAL,
                "tensor-core context attention: bad context size");
  ARTAB_REQUIRE(((uintptr_t)a.q % 16) == 0 && ((uintptr_t)a.k_ctx % 16) == 0 && ((uintptr_t)a.v_ctx % 16) == 0,
                ARTAB_EINVAL, "tensor-core context attention: q / k / v must be 16-byte aligned");
  const int D = a.n_heads * DH;
  CUtensorMap tq, tk, tv;
  int rc = make_map_2d(&tq, a.q, (uint64_t)D, (uint64_t)a.rows, (uint64_t)D * 2, DH, BM, CU_TENSOR_MAP_SWIZZLE_64B, "q");
  if (rc) return rc;
  const uint64_t gh = (uint64_t)a.n_groups * a.n_heads;
  rc = make_map_2d(&tk, a.k_ctx, DH, gh * a.n_ctx_pad, DH * 2, DH, BN, CU_TENSOR_MAP_SWIZZLE_64B, "k_ctx");
  if (rc) return rc;
  rc = make_map_2d(&tv, a.v_ctx, (uint64_t)a.n_ctx_pad, gh * 2 * DH, (uint64_t)a.n_ctx_pad * 2, 64, 2 * DH,
                   CU_TENSOR_MAP_SWIZZLE_128B, "v_ctx");
  if (rc) return rc;

  // two CTAs per SM at most: each holds 256 of the SM's 512 TMEM columns
  const size_t smem = 100 * 1024;
  static_assert(sizeof(Smem) + 1024 <= 100 * 1024, "shared-memory plan exceeds the request");
  static SmemConfig configured;
  {
    const cudaError_t e = configured.ensure(ctx_attn_tc_kernel, smem, true);
    ARTAB_REQUIRE(e == cudaSuccess, ARTAB_ELAUNCH, "ctx_attn_tc_kernel: shared memory refused: %s",
                  cudaGetErrorString(e));
  }
  TcParams p;
  p.rows = a.rows;
  p.rows_per_group = a.rows_per_group;
  p.n_groups = a.n_groups;
  p.n_heads = a.n_heads;
  p.n_ctx = a.n_ctx;
  p.n_ctx_pad = a.n_ctx_pad;
  p.n_splits = a.n_splits;
  p.scale_log2e = a.scale * kLog2e;
  p.out_lane_major = a.out_lane_major && a.n_splits == 1;
  p.kv_stable = a.kv_stable;
  p.out = a.out;
  p.lse = a.lse;
  p.status = a.status;
  p.wait_cycles = debug_wait_cycles() > 0 ? debug_wait_cycles() : kWaitCycles;
  p.drop_score_commits = debug_drop_score_commits();
  const int rows_in_group = a.n_groups == 1 ? a.rows : a.rows_per_group;
  dim3 grid((rows_in_group + BM - 1) / BM, a.n_heads, a.n_groups * a.n_splits);
  prof_begin(PROF_CTX, s);
  ARTAB_STAMP_ATTACH();
  const cudaError_t le = launch_dependent(ctx_attn_tc_kernel, grid, dim3(kThreads), smem, s, tq, tk, tv, p);
  prof_end(s);
  ARTAB_REQUIRE(le == cudaSuccess, ARTAB_ELAUNCH, "ctx_attn_tc_kernel: %s", cudaGetErrorString(le));
  count_launch();
  return check_launch("ctx_attn_tc_kernel");
}

}  // namespace artab
